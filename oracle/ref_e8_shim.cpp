// TEST INFRASTRUCTURE ONLY. Compiles the reference's own E8 decode and cell hash
// (cpp/src/neighbors/octex/detail/e8.cuh of hpdic/octex) for the host, from where the reference
// sources lie, so that the restatement in e8_port.hpp can be pinned against the real thing and so
// that golden vectors can be generated. The header is plain C++ once three CUDA keywords are
// defined away; the include path is given on the command line by the Makefile. No reference
// source is copied into this repository.
#define __device__
#define __forceinline__ inline
#define __constant__ static const
#include <math.h>
#include "e8.cuh"

#include <cstdint>

extern "C" {

int ref_e8_point(const float* x, int64_t n_blocks, float* p)
{
  for (int64_t i = 0; i < n_blocks; i++)
    cuvs::neighbors::octex::detail::e8_point(x + 8 * i, p + 8 * i);
  return 0;
}

int ref_cell_code(const float* y, int64_t n, int32_t b, float inv_f, int64_t* h)
{
  for (int64_t i = 0; i < n; i++)
    h[i] = cuvs::neighbors::octex::detail::e8b_hash64(y + i * 8 * b, b, inv_f);
  return 0;
}
}
