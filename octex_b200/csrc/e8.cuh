// E8 lattice decode and 64-bit cell code, shared by every kernel that needs a cell.
//
// Semantics follow the reference's device functions (hpdic/octex,
// cpp/src/neighbors/octex/detail/e8.cuh:25-85): E8 = D8 u (D8 + 1/2); the nearest D8 point is the
// coordinate-wise rounding (half to even) with the worst-rounded coordinate moved one step when
// the sum is odd; the nearer of the two cosets wins, the integer one on a tie; the code is a
// prime-weighted sum of the doubled coordinates per block, chained over blocks with the 64-bit
// golden-ratio constant and finished by two xor-shift-multiply steps.
//
// Floating-point contract: every operation is written with explicit round-to-nearest intrinsics so
// that the compiler cannot fuse or reorder them; the only fused multiply-adds are the two
// squared-error accumulations, one per coordinate in coordinate order. The CPU checker of this
// repository states the same contract, which makes codes comparable bit for bit.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace octex_b200 {

static __device__ __constant__ unsigned long long kCellPrimes[8] = {1000003ULL,
                                                              998244353ULL,
                                                              1000000007ULL,
                                                              2147483647ULL,
                                                              1099511627791ULL,
                                                              4398042316799ULL,
                                                              70368744177643ULL,
                                                              1125899906842597ULL};
constexpr unsigned long long kGolden = 0x9E3779B97F4A7C15ULL;

/// Nearest D8 point of v[0..8) into out[0..8).
__device__ __forceinline__ void nearest_d8(const float (&v)[8], float (&out)[8])
{
  float total = 0.f, worst = -1.f, worst_e = 0.f;
  int worst_at = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float r = rintf(v[i]);
    out[i]        = r;
    total         = __fadd_rn(total, r);
    const float e = __fsub_rn(v[i], r);
    const float a = fabsf(e);
    if (a > worst) {
      worst    = a;
      worst_at = i;
      worst_e  = e;
    }
  }
  // total is an integer-valued float: odd <=> its remainder by 2 is non-zero
  if (fmodf(total, 2.f) != 0.f) {
    const float step = worst_e >= 0.f ? 1.f : -1.f;
#pragma unroll
    for (int i = 0; i < 8; i++)
      if (i == worst_at) out[i] = __fadd_rn(out[i], step);
  }
}

/// Nearest E8 point of v[0..8) into out[0..8) (coordinates in Z/2).
__device__ __forceinline__ void nearest_e8(const float (&v)[8], float (&out)[8])
{
  float ints[8], halves[8], moved[8];
#pragma unroll
  for (int i = 0; i < 8; i++)
    moved[i] = __fsub_rn(v[i], 0.5f);
  nearest_d8(v, ints);
  nearest_d8(moved, halves);
  float err_i = 0.f, err_h = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    halves[i]     = __fadd_rn(halves[i], 0.5f);
    const float a = __fsub_rn(v[i], ints[i]);
    const float c = __fsub_rn(v[i], halves[i]);
    err_i         = __fmaf_rn(a, a, err_i);
    err_h         = __fmaf_rn(c, c, err_h);
  }
  const bool take_ints = err_i <= err_h;
#pragma unroll
  for (int i = 0; i < 8; i++)
    out[i] = take_ints ? ints[i] : halves[i];
}

/// Prime-weighted sum of the doubled coordinates of the E8 point nearest to v (one block).
__device__ __forceinline__ unsigned long long block_code(const float (&v)[8])
{
  float p[8];
  nearest_e8(v, p);
  unsigned long long hb = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const long long twice = static_cast<long long>(__fmul_rn(2.f, p[i]));
    hb += static_cast<unsigned long long>(twice) * kCellPrimes[i];
  }
  return hb;
}

/// Final mixing of a chained block code.
__device__ __forceinline__ long long finish_code(unsigned long long h)
{
  long long s = static_cast<long long>(h);
  s           = static_cast<long long>(static_cast<unsigned long long>(s ^ (s >> 31)) * kGolden);
  return s ^ (s >> 29);
}

/// Cell code of the 8*B coordinates y scaled by inv_f.
template <int B>
__device__ __forceinline__ long long cell_code(const float (&y)[8 * B], float inv_f)
{
  unsigned long long h = 0;
#pragma unroll
  for (int j = 0; j < B; j++) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++)
      v[i] = __fmul_rn(y[8 * j + i], inv_f);
    const unsigned long long hb = block_code(v);
    h                           = (j == 0) ? hb : h * kGolden + hb;
  }
  return finish_code(h);
}

// ---------------------------------------------------------------------------------------------
// The same decode for coordinates known to be small: every |v[i]| < kTameLimit (and no NaN). Under
// that bound each step below gives the value the general code gives, so the codes are identical;
// what changes is the instruction mix: no conversion-unit instructions and no branches.
//   * rint(x) = (x + 1.5 * 2^23) - 1.5 * 2^23 in round-to-nearest arithmetic (ties to even), exact
//     for |x| < 2^22. A rounded -0 comes out as +0, which no later step can tell apart.
//   * the sum of the rounded coordinates is an exact integer below 2^24: it is odd iff half of it is
//     not an integer.
//   * 2 p + 1.5 * 2^23 is exact, and its bit pattern is 0x4B400000 + 2 p as an integer: the weighted
//     sum runs over these unsigned words and the constant part is taken off at the end (all modulo
//     2^64, as in the general code).
constexpr float kTameLimit = 1048576.f;  // 2^20
constexpr float kRintMagic = 12582912.f;  // 1.5 * 2^23, bit pattern 0x4B400000

__host__ __device__ constexpr unsigned long long cell_prime(int i)
{
  return i == 0   ? 1000003ULL
         : i == 1 ? 998244353ULL
         : i == 2 ? 1000000007ULL
         : i == 3 ? 2147483647ULL
         : i == 4 ? 1099511627791ULL
         : i == 5 ? 4398042316799ULL
         : i == 6 ? 70368744177643ULL
                  : 1125899906842597ULL;
}

__device__ __forceinline__ float rint_tame(float x)
{
  return __fsub_rn(__fadd_rn(x, kRintMagic), kRintMagic);
}

__device__ __forceinline__ void nearest_d8_tame(const float (&v)[8], float (&out)[8])
{
  out[0]        = rint_tame(v[0]);
  float total   = out[0];
  float worst_e = __fsub_rn(v[0], out[0]);
  int worst_at  = 0;
#pragma unroll
  for (int i = 1; i < 8; i++) {
    const float r = rint_tame(v[i]);
    out[i]        = r;
    total         = __fadd_rn(total, r);
    const float e = __fsub_rn(v[i], r);
    if (fabsf(e) > fabsf(worst_e)) {  // strictly larger: the first of equal errors stays
      worst_at = i;
      worst_e  = e;
    }
  }
  const float half = __fmul_rn(total, 0.5f);
  const bool odd   = rint_tame(half) != half;
  const float step = odd ? (worst_e >= 0.f ? 1.f : -1.f) : 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++)
    out[i] = __fadd_rn(out[i], i == worst_at ? step : 0.f);
}

__device__ __forceinline__ unsigned long long block_code_tame(const float (&v)[8])
{
  float ints[8], halves[8], moved[8];
#pragma unroll
  for (int i = 0; i < 8; i++)
    moved[i] = __fsub_rn(v[i], 0.5f);
  nearest_d8_tame(v, ints);
  nearest_d8_tame(moved, halves);
  float err_i = 0.f, err_h = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    halves[i]     = __fadd_rn(halves[i], 0.5f);
    const float a = __fsub_rn(v[i], ints[i]);
    const float c = __fsub_rn(v[i], halves[i]);
    err_i         = __fmaf_rn(a, a, err_i);
    err_h         = __fmaf_rn(c, c, err_h);
  }
  const bool take_ints = err_i <= err_h;
  unsigned long long hb = 0, primes = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float p    = take_ints ? ints[i] : halves[i];
    const unsigned u = __float_as_uint(__fmaf_rn(2.f, p, kRintMagic));
    hb += static_cast<unsigned long long>(u) * cell_prime(i);
    primes += cell_prime(i);
  }
  return hb - 0x4B400000ULL * primes;
}

/// cell_code for coordinates with |y[i] * inv_f| < kTameLimit: the same code, fewer instructions.
template <int B>
__device__ __forceinline__ long long cell_code_tame(const float (&y)[8 * B], float inv_f)
{
  unsigned long long h = 0;
#pragma unroll
  for (int j = 0; j < B; j++) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++)
      v[i] = __fmul_rn(y[8 * j + i], inv_f);
    const unsigned long long hb = block_code_tame(v);
    h                           = (j == 0) ? hb : h * kGolden + hb;
  }
  return finish_code(h);
}

}  // namespace octex_b200
