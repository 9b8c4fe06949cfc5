// Stand-in (see ../../device_uvector.hpp): bins are accepted and ignored; the
// CUDA stream-ordered pool already caches freed blocks.
#pragma once
#include <cstddef>
namespace rmm { namespace mr {
template <typename Upstream>
class binning_memory_resource {
 public:
  explicit binning_memory_resource(Upstream *) {}
  void add_bin(std::size_t) {}
};
}}
