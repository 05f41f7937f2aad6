// Error handling and owned device memory shared by the host code of the library.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>

namespace octex_b200 {

/// Every failure of the library is one of these; the C boundary turns it into an error code and
/// a per-thread message (the reference does the same with raft::exception,
/// c/src/core/exceptions.hpp:17-33 of hpdic/octex).
struct error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

#define OCTEX_EXPECTS(cond, msg)                       \
  do {                                                 \
    if (!(cond)) throw ::octex_b200::error(msg);       \
  } while (0)

#define OCTEX_CUDA_TRY(call)                                                              \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess) {                                                              \
      cudaGetLastError();                                                                 \
      throw ::octex_b200::error(std::string("octex: CUDA error at ") + __FILE__ + ":" +   \
                                std::to_string(__LINE__) + ": " + cudaGetErrorString(e_)); \
    }                                                                                     \
  } while (0)

/// Device memory owned on one GPU and freed on it.
struct dbuf {
  void* ptr   = nullptr;
  size_t size = 0;
  int device  = -1;

  dbuf() = default;
  dbuf(int dev, size_t bytes) : size(bytes), device(dev)
  {
    if (bytes == 0) return;
    OCTEX_CUDA_TRY(cudaSetDevice(dev));
    OCTEX_CUDA_TRY(cudaMalloc(&ptr, bytes));
  }
  dbuf(dbuf const&)                    = delete;
  auto operator=(dbuf const&) -> dbuf& = delete;
  dbuf(dbuf&& o) noexcept { swap(o); }
  auto operator=(dbuf&& o) noexcept -> dbuf&
  {
    swap(o);
    return *this;
  }
  ~dbuf()
  {
    if (ptr == nullptr || !owned) return;
    if (host) {
      cudaFreeHost(ptr);
      return;
    }
    int cur = 0;
    cudaGetDevice(&cur);
    cudaSetDevice(device);
    cudaFree(ptr);
    cudaSetDevice(cur);
  }
  void swap(dbuf& o) noexcept
  {
    std::swap(ptr, o.ptr);
    std::swap(size, o.size);
    std::swap(device, o.device);
    std::swap(owned, o.owned);
    std::swap(host, o.host);
  }
  /// Page-locked host memory every GPU can read through the same pointer (the host tier of an
  /// index array: cpp/src/neighbors/octex/detail/index_impl.hpp:69-113 of the reference).
  static auto pinned(int dev, size_t bytes) -> dbuf
  {
    dbuf b;
    b.size   = bytes;
    b.device = dev;
    b.host   = true;
    if (bytes != 0)
      OCTEX_CUDA_TRY(cudaHostAlloc(&b.ptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
    return b;
  }
  /// A view of memory owned by the caller (arrays attached without a copy).
  static auto borrow(int dev, const void* p, size_t bytes) -> dbuf
  {
    dbuf b;
    b.ptr    = const_cast<void*>(p);
    b.size   = bytes;
    b.device = dev;
    b.owned  = false;
    return b;
  }
  template <typename T>
  [[nodiscard]] auto as() const -> T*
  {
    return static_cast<T*>(ptr);
  }
  bool owned = true;
  bool host  = false;
};

}  // namespace octex_b200
