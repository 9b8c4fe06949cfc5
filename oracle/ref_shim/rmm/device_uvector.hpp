// Stand-in for rmm::device_uvector used only to compile the unmodified
// reference sources into oracle/_ref (test infrastructure). Written for this
// repository; it is not RMM. Semantics the reference relies on: uninitialised
// storage on a stream, move-only, resize that preserves the common prefix.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <utility>

namespace rmm {

struct cuda_stream_view {
  cudaStream_t s = cudaStreamLegacy;
  cuda_stream_view() = default;
  cuda_stream_view(cudaStream_t st) : s(st) {}
  operator cudaStream_t() const { return s; }
  cudaStream_t value() const { return s; }
  bool operator==(const cuda_stream_view &o) const { return s == o.s; }
  bool operator!=(const cuda_stream_view &o) const { return s != o.s; }
};

template <typename T>
class device_uvector {
 public:
  using value_type = T;
  using size_type = std::size_t;
  using pointer = T *;
  using const_pointer = const T *;

  device_uvector(std::size_t size, cuda_stream_view stream) : stream_(stream) {
    allocate(size);
  }
  ~device_uvector() { release(); }
  device_uvector(const device_uvector &) = delete;
  device_uvector &operator=(const device_uvector &) = delete;
  device_uvector(device_uvector &&o) noexcept
      : data_(o.data_), size_(o.size_), cap_(o.cap_), stream_(o.stream_) {
    o.data_ = nullptr;
    o.size_ = o.cap_ = 0;
  }
  device_uvector &operator=(device_uvector &&o) noexcept {
    if (this != &o) {
      release();
      data_ = o.data_;
      size_ = o.size_;
      cap_ = o.cap_;
      stream_ = o.stream_;
      o.data_ = nullptr;
      o.size_ = o.cap_ = 0;
    }
    return *this;
  }

  void resize(std::size_t new_size, cuda_stream_view stream) {
    stream_ = stream;
    if (new_size <= cap_) {
      size_ = new_size;
      return;
    }
    T *old = data_;
    std::size_t old_size = size_;
    data_ = nullptr;
    allocate(new_size);
    if (old) {
      if (old_size) cudaMemcpyAsync(data_, old, old_size * sizeof(T), cudaMemcpyDeviceToDevice, stream_.s);
      cudaFreeAsync(old, stream_.s);
    }
  }

  T *data() noexcept { return data_; }
  const T *data() const noexcept { return data_; }
  std::size_t size() const noexcept { return size_; }
  bool is_empty() const noexcept { return size_ == 0; }
  cuda_stream_view stream() const noexcept { return stream_; }
  T *begin() noexcept { return data_; }
  T *end() noexcept { return data_ + size_; }
  const T *begin() const noexcept { return data_; }
  const T *end() const noexcept { return data_ + size_; }

 private:
  void allocate(std::size_t n) {
    size_ = cap_ = n;
    if (n) cudaMallocAsync(reinterpret_cast<void **>(&data_), n * sizeof(T), stream_.s);
  }
  void release() {
    if (data_) cudaFreeAsync(data_, stream_.s);
    data_ = nullptr;
    size_ = cap_ = 0;
  }
  T *data_ = nullptr;
  std::size_t size_ = 0, cap_ = 0;
  cuda_stream_view stream_;
};

}  // namespace rmm
