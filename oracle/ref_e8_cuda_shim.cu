// TEST INFRASTRUCTURE ONLY. The reference's own E8 decode and cell hash
// (cpp/src/neighbors/octex/detail/e8.cuh of hpdic/octex) compiled as device code, with nvcc's
// default flags as the reference's build uses them, behind one host function. It lets a GPU test
// compare the codes of this repository's kernels with the codes the reference's device function
// gives on the same GPU. The header is included from where the reference sources lie; nothing of
// it is copied here.
#include "e8.cuh"

#include <cuda_runtime.h>

#include <cstdint>

namespace {
__global__ void ref_codes_kernel(const float* y, int64_t n, int b, float inv_f, long long* h)
{
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i < n) h[i] = cuvs::neighbors::octex::detail::e8b_hash64(y + i * 8 * b, b, inv_f);
}
}  // namespace

// Host pointers in and out; returns 0, or the CUDA error code.
extern "C" int ref_cuda_cell_code(const float* y, int64_t n, int32_t b, float inv_f, int64_t* h)
{
  float* dy     = nullptr;
  long long* dh = nullptr;
  cudaError_t e = cudaMalloc(&dy, sizeof(float) * n * 8 * b);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMalloc(&dh, sizeof(long long) * n);
  if (e == cudaSuccess) e = cudaMemcpy(dy, y, sizeof(float) * n * 8 * b, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) {
    ref_codes_kernel<<<static_cast<unsigned>((n + 255) / 256), 256>>>(dy, n, b, inv_f, dh);
    e = cudaDeviceSynchronize();
  }
  if (e == cudaSuccess) e = cudaMemcpy(h, dh, sizeof(long long) * n, cudaMemcpyDeviceToHost);
  cudaFree(dy);
  cudaFree(dh);
  return static_cast<int>(e);
}
