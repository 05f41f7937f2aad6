// TEST INFRASTRUCTURE ONLY. CPU restatement of the E8 decode and cell hash of the octex search
// path. Nothing outside tests/, the smoke check and the CPU-baseline leg of the benchmark may
// call it. The shipped library never links or loads this file.
//
// Follows the reference's device functions:
//   d8          cpp/src/neighbors/octex/detail/e8.cuh:25-42
//   e8_point    cpp/src/neighbors/octex/detail/e8.cuh:45-63
//   e8b_hash64  cpp/src/neighbors/octex/detail/e8.cuh:66-85
//   kPrimes     cpp/src/neighbors/octex/detail/e8.cuh:13-20,  kMix e8.cuh:21
//
// Floating-point contract (shared with the CUDA path of this repository so both are bit-equal):
// the two squared errors that choose between the integer and the half-integer coset are
// accumulated with one fused multiply-add per coordinate, in coordinate order.
#pragma once

#include <cmath>
#include <cstdint>

namespace octex_oracle {

static const uint64_t kCellPrimes[8] = {1000003ULL,
                                        998244353ULL,
                                        1000000007ULL,
                                        2147483647ULL,
                                        1099511627791ULL,
                                        4398042316799ULL,
                                        70368744177643ULL,
                                        1125899906842597ULL};
static const uint64_t kGolden = 0x9E3779B97F4A7C15ULL;

// Nearest point of D8 (integer coordinates, even sum) to v[0..8).
inline void nearest_d8(const float* v, float* out)
{
  float total    = 0.f;
  float worst    = -1.f;
  float worst_e  = 0.f;
  int worst_at   = 0;
  for (int i = 0; i < 8; i++) {
    float r = std::rint(v[i]);  // round half to even
    out[i]  = r;
    total += r;
    float e = v[i] - r;
    if (std::fabs(e) > worst) {  // strict: the first coordinate wins a tie
      worst    = std::fabs(e);
      worst_at = i;
      worst_e  = e;
    }
  }
  if (std::fmod(total, 2.f) != 0.f) out[worst_at] += (worst_e >= 0.f ? 1.f : -1.f);
}

// Nearest point of E8 = D8 ∪ (D8 + ½) to v[0..8); the integer coset wins an exact tie.
inline void nearest_e8(const float* v, float* out)
{
  float ints[8], halves[8], moved[8];
  for (int i = 0; i < 8; i++)
    moved[i] = v[i] - 0.5f;
  nearest_d8(v, ints);
  nearest_d8(moved, halves);
  float err_i = 0.f, err_h = 0.f;
  for (int i = 0; i < 8; i++) {
    halves[i] += 0.5f;
    float a = v[i] - ints[i];
    float c = v[i] - halves[i];
    err_i   = std::fma(a, a, err_i);
    err_h   = std::fma(c, c, err_h);
  }
  const bool take_ints = err_i <= err_h;
  for (int i = 0; i < 8; i++)
    out[i] = take_ints ? ints[i] : halves[i];
}

// 64-bit code of the E8^b cell of y * inv_f (y: 8b coordinates).
inline int64_t cell_code(const float* y, int b, float inv_f)
{
  uint64_t h = 0;
  for (int j = 0; j < b; j++) {
    float v[8], p[8];
    for (int i = 0; i < 8; i++)
      v[i] = y[8 * j + i] * inv_f;
    nearest_e8(v, p);
    uint64_t hb = 0;
    for (int i = 0; i < 8; i++) {
      int64_t twice = static_cast<int64_t>(2.f * p[i]);
      hb += static_cast<uint64_t>(twice) * kCellPrimes[i];
    }
    h = (j == 0) ? hb : h * kGolden + hb;
  }
  int64_t s = static_cast<int64_t>(h);
  s         = static_cast<int64_t>(static_cast<uint64_t>(s ^ (s >> 31)) * kGolden);
  return s ^ (s >> 29);
}

}  // namespace octex_oracle
