// Pieces shared by the tensor-core kernels (sm_100a): bounded mbarrier waits, TMA tile loads, the
// shared-memory descriptor of a 128-byte-swizzled K-major operand tile, tcgen05.mma / commit, and
// the host-side tensor maps of row-major fp16 matrices.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace octex_b200::kernels {

constexpr int kTileK          = 64;        // halves per operand row in a stage (128 bytes, the swizzle span)
constexpr uint32_t kSpinLimit = 1u << 21;  // polls of an mbarrier before giving up

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

/// Wait for the phase with the given parity; false when the poll limit ran out or *give_up
/// (may be null) became non-zero.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* give_up = nullptr)
{
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (give_up != nullptr && *give_up != 0) return false;
    uint32_t ok;
    asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(addr), "r"(parity)
      : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
    ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
    : "memory");
}

/// Shared-memory matrix descriptor of a K-major operand tile written by TMA with the 128-byte
/// swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(const void* tile)
{
  const uint64_t addr = (smem_u32(tile) & 0x3FFFFu) >> 4;
  return addr | (uint64_t{1} << 16)      // leading byte offset (unused with a swizzle): 16 bytes
         | (uint64_t{1024 >> 4} << 32)   // stride byte offset: 1024 bytes between 8-row groups
         | (uint64_t{1} << 46)           // descriptor version of this architecture
         | (uint64_t{2} << 61);          // layout: 128-byte swizzle
}

/// D (fp32, TMEM) (+)= A (fp16, K-major) x B^T (fp16, K-major), 128 x 128 x 16.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                         uint32_t accumulate)
{
  asm volatile(
    "{\n\t"
    ".reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
    "}"
    ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
    : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}


using encode_fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

inline auto encoder() -> encode_fn
{
  static encode_fn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q{};
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      cudaGetLastError();
      throw std::runtime_error("octex: the driver has no cuTensorMapEncodeTiled");
    }
    fn = reinterpret_cast<encode_fn>(p);
  }
  return fn;
}

/// Tensor map of a row-major fp16 matrix [rows, ld] read in boxes of rows_box x 64 halves with the
/// 128-byte swizzle; rows and columns beyond the matrix read as zero.
inline void make_map(void* out, const __half* base, int64_t rows, int64_t ld, int rows_box)
{
  CUtensorMap map;
  const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(__half)};
  const cuuint32_t box[2]     = {kTileK, static_cast<cuuint32_t>(rows_box)};
  const cuuint32_t estr[2]    = {1, 1};
  CUresult r = encoder()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("octex: cuTensorMapEncodeTiled failed (" + std::to_string(static_cast<int>(r)) + ")");
  static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
  std::memcpy(out, &map, sizeof(map));
}


}  // namespace octex_b200::kernels
