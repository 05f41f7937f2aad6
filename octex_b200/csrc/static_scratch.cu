// Cell codes of a batch of queries without any allocation: octexB200QueryCodesStatic.
//
// Who this is for. Some callers must not allocate device memory at the point where they need the
// codes: services whose whole device memory was handed to one arena at start-up, so that a later
// cudaMalloc fails or breaks the rules of the process; latency-bound loops that cannot afford the
// device-wide synchronisation a cudaMalloc / cudaFree pair implies; and code that runs while a
// stream capture is open elsewhere in the process, where cudaMalloc is not allowed. The normal
// search keeps its intermediates
// in buffers it allocates when a plan is made; this entry point keeps them in a fixed array that
// is part of the library image instead, so the call itself never allocates.
//
// The price: the array below exists once per GPU that loads the library (kScratchBytes of device
// memory per GPU until the process exits, used or not), a batch must fit in it, every call on a
// GPU uses the same bytes, and nothing is remembered between calls except those bytes.

#include "search_impl.hpp"

#include <octex_b200.h>

#include <algorithm>
#include <string>

namespace {

/// Upper bound of the intermediates of one call, in bytes. A batch of m queries needs
/// m * (2 * ldu + 4 * sketch_width + 2 * 8 * blocks * copies) bytes: its centred fp16 queries, its
/// sketch-space queries and its fp16 projected coordinates.
constexpr size_t kScratchBytes = size_t{32} << 20;

/// The intermediates of octexB200QueryCodesStatic. In host code this name is only a handle for
/// cudaGetSymbolAddress; the address kernels can use is looked up in scratch_of_current_device().
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

/// Device address of the static array on the current device. Asked for at every call: the
/// address belongs to the current device's context (it changes after a cudaDeviceReset), the lookup
/// is cheap once the module is loaded, and the first lookup on a device loads the module there,
/// which is why the first call on a device should happen outside of any stream capture.
auto scratch_of_current_device() -> unsigned char*
{
  void* p       = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw octex_b200::error(std::string("octex: cudaGetSymbolAddress of the static scratch: ") +
                            cudaGetErrorString(e));
  }
  OCTEX_EXPECTS(p != nullptr, "octex: the static scratch has no device address");
  return static_cast<unsigned char*>(p);
}

auto align_up(size_t v, size_t a) -> size_t { return (v + a - 1) / a * a; }

}  // namespace

extern "C" cuvsError_t octexB200QueryCodesStatic(cuvsOctexIndex_t index, const float* queries,
                                                 int64_t n_queries, int64_t* codes, void* stream)
{
  try {
    using namespace octex_b200;
    OCTEX_EXPECTS(index != nullptr && index->addr != 0, "octex: the index is empty (load it first)");
    auto& ix      = reinterpret_cast<octex_b200::index*>(index->addr)->impl();
    auto const& p = ix.part;
    OCTEX_EXPECTS(n_queries >= 0, "octex: a negative number of queries");
    if (n_queries == 0) {
      cuvsSetLastErrorText(nullptr);
      return CUVS_SUCCESS;
    }
    OCTEX_EXPECTS(queries != nullptr && codes != nullptr, "octex: a NULL array");
    int dev = -1;
    OCTEX_CUDA_TRY(cudaGetDevice(&dev));
    OCTEX_EXPECTS(dev == p.device, "octex: the current device is not the device of the index");
    OCTEX_EXPECTS(p.copies == ix.copies,
                  "octex: this process holds " + std::to_string(p.copies) + " of the index's " +
                    std::to_string(ix.copies) + " copies (shard placement over several processes); "
                    "the static-scratch call answers for whole indexes only");
    const int D = static_cast<int>(ix.dim), sw = ix.sketch_width;
    const int L = static_cast<int>(ix.spacings.size());
    const int N = 8 * ix.blocks * p.copies;
    // carve the array: centred fp16 queries | sketch-space queries | projected coordinates
    const size_t m       = static_cast<size_t>(n_queries);
    const size_t qh_off  = 0;
    const size_t qs_off  = align_up(qh_off + m * p.ldu * sizeof(__half), 256);
    const size_t y_off   = align_up(qs_off + m * sw * sizeof(float), 256);
    const size_t need    = y_off + m * N * sizeof(__half);
    if (need > kScratchBytes) {
      const size_t per = static_cast<size_t>(p.ldu) * 2 + static_cast<size_t>(sw) * 4 + static_cast<size_t>(N) * 2;
      throw octex_b200::error("octex: " + std::to_string(n_queries) +
                              " queries need " + std::to_string(need) +
                              " bytes of intermediates, the static scratch holds " +
                              std::to_string(kScratchBytes) + " (at most about " +
                              std::to_string((kScratchBytes - 512) / per) +
                              " queries per call for this index)");
    }
    OCTEX_EXPECTS(n_queries <= 0x7fffffff / std::max(N, 1), "octex: too many queries for one call");
    unsigned char* base = scratch_of_current_device();
    auto* qh            = reinterpret_cast<__half*>(base + qh_off);
    auto* qs            = reinterpret_cast<float*>(base + qs_off);
    auto* Y             = reinterpret_cast<__half*>(base + y_off);
    auto s              = static_cast<cudaStream_t>(stream);
    // every byte the three kernels read from the array is written by this call first (the zero
    // padding of the fp16 queries included), so nothing has to be cleared between calls
    kernels::center_sketch(queries, p.mean.as<float>(), p.basis.as<float>(), static_cast<int>(m), D,
                           sw, qh, p.ldu, qs, s);
    kernels::project_ordered(qh, p.ldu, p.ut.as<__half>(), p.ldu, p.shift.as<__half>(),
                             static_cast<int>(m), N, D, Y, s);
    kernels::decode_codes(Y, static_cast<int64_t>(m) * p.copies, p.copies, ix.blocks, L,
                          p.inv_f.as<float>(), nullptr, reinterpret_cast<long long*>(codes), s);
    OCTEX_CUDA_TRY(cudaPeekAtLastError());
    cuvsSetLastErrorText(nullptr);
    return CUVS_SUCCESS;
  } catch (std::exception const& e) {
    cuvsSetLastErrorText(e.what());
    return CUVS_ERROR;
  }
}
