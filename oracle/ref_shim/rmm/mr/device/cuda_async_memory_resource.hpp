// Stand-in (see ../../device_uvector.hpp): the stream-ordered CUDA allocator
// is used directly by the device_uvector stand-in, so this type carries nothing.
#pragma once
namespace rmm { namespace mr {
class cuda_async_memory_resource {};
}}
