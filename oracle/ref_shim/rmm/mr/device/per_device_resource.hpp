// Stand-in (see ../../device_uvector.hpp).
#pragma once
namespace rmm { namespace mr {
template <typename R>
inline void set_current_device_resource(R *) {}
inline void set_current_device_resource(decltype(nullptr)) {}
}}
