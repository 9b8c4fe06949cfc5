// Stand-in (see ../../device_uvector.hpp): the stream-ordered CUDA allocator
// is used directly by the device_uvector stand-in. What this type does keep of
// RMM's cuda_async_memory_resource is its pool behaviour: RMM raises the
// release threshold of the device's default memory pool so that freed blocks
// stay in the pool across synchronisations instead of going back to the
// driver; constructing the stand-in does the same.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
namespace rmm { namespace mr {
class cuda_async_memory_resource {
 public:
  cuda_async_memory_resource() {
    int device = 0;
    cudaMemPool_t pool = nullptr;
    if (cudaGetDevice(&device) == cudaSuccess && cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
      std::uint64_t keep = UINT64_MAX;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
  }
};
}}
