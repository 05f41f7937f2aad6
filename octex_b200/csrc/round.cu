// One round of the search per query block (sm_100a): gather, dedup, sketch scoring, selection,
// exact rerank and merge into the kept list in one kernel; for waves the choice of the start points
// comes first in the same kernel. A query's candidates stay in shared memory from the first list
// entry to the kept list.
//
// Semantics follow the reference's per-step kernels (hpdic/octex,
// cpp/src/neighbors/octex/detail/search_kernels.cuh): gather_kernel :138-253, select_smallest
// :259-322, exact_distances :325-342, load_keys / bitonic_sort / store_keys :345-415,
// rerank_keep_kernel :421-467, sketch_keep_kernel :471-508, merge_kept_kernel :517-564,
// pick_starts_kernel :571-631, final_rerank_kernel :634-669. What differs is how the work is laid
// out: the kept list is never fully re-sorted (the best KO keys are selected by radix passes and
// only those are sorted), candidates already in the kept list are not reranked again (their key is
// already there), and every thread keeps several independent loads in flight.

#include "kernels.hpp"

#include <algorithm>
#include <cfloat>
#include <cmath>

namespace octex_b200::kernels {

namespace {

constexpr unsigned kIdHash          = 2654435761u;
constexpr unsigned long long kNoKey = ~0ULL;

/// Offsets (in 4-byte words) of the regions of a round block's shared memory.
struct round_layout {
  int table, cand, dist, pool, sorted, sid, sdv, qv, sc, fq, st, len, hist, wsum, ctrl, kid, kd, words;
  __host__ __device__ explicit round_layout(const round_args& a)
  {
    const int in_smem = a.cand_global == nullptr ? a.nmax : 0;
    const int rm      = a.sketch_rank ? a.KO : a.R;
    int at            = 0;
    auto take         = [&](int n) {
      int o = at;
      at += (n + 3) & ~3;  // keep every region 16-byte aligned
      return o;
    };
    // Two regions are used twice. The sketch distances are written where the hash set of the gather
    // was (the set is dead once the ids are collected; the filter of kept ids, which builds a small
    // set there again, starts after the selection has copied out the distances it needs). The keys of
    // the merge are written where the candidates were (dead after the selection).
    const int pool_words = 2 * (a.KO + rm);
    const int sort_words = a.P > 32 ? 4 * a.P : 128;  // 2 P keys, 64 at least (the one-warp sort)
    table  = take(a.ht_slots > in_smem ? a.ht_slots : in_smem);
    dist   = table;
    cand   = take(in_smem > pool_words + sort_words ? in_smem : pool_words + sort_words);
    pool   = cand;
    sorted = cand + pool_words;
    sid    = take(rm);
    sdv    = take(rm);
    // first round: 16-bit weights of the integer sketch distance (two per word) and its per-query
    // constants (-2 alpha, sum of q^2); waves: the sketch-space query and the scales as floats
    qv     = take(a.sw);
    sc     = take(a.sw);
    fq     = take((a.D + 63) & ~63);  // in 64-element steps (query_slot)
    st     = take(a.nseg);
    len    = take(a.nseg);
    hist   = take(256);
    wsum   = take(20);
    ctrl   = take(8);
    kid    = take(a.KO);
    kd     = take(a.KO);
    words  = at;
  }
};

/// Home slot of an id in a set of `slots` (any size): the high word of hash * slots.
__device__ __forceinline__ unsigned home_slot(int id, int slots)
{
  return __umulhi(static_cast<unsigned>(id) * kIdHash, static_cast<unsigned>(slots));
}

/// Exclusive prefix of v over the block (kThreads threads); total = the sum. wsum: kThreads / 32 + 1
/// words.
template <int kThreads = kRoundThreads>
__device__ __forceinline__ int block_scan(int v, int* wsum, int& total)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int nw = kThreads / 32;
  int inc          = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += u;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const int w = lane < nw ? wsum[lane] : 0;
    int winc    = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += u;
    }
    if (lane < nw) wsum[lane] = winc - w;
    if (lane == nw - 1) wsum[nw] = winc;
  }
  __syncthreads();
  const int out = wsum[warp] + inc - v;
  total         = wsum[nw];
  __syncthreads();
  return out;
}

/// (distance bits << 32) | id: the total order of every kept list (search_kernels.cuh:365-368).
__device__ __forceinline__ unsigned long long rank_key(float d, unsigned id)
{
  return (static_cast<unsigned long long>(__float_as_uint(d)) << 32) | id;
}

/// Ascending bitonic sort of P (power of two) 64-bit keys in shared memory.
__device__ __forceinline__ void bitonic_sort(unsigned long long* key, int P)
{
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < P; i += blockDim.x) {
        const int j = i ^ stride;
        if (j > i) {
          const bool up              = (i & size) == 0;
          const unsigned long long a = key[i], b = key[j];
          if ((a > b) == up) {
            key[i] = b;
            key[j] = a;
          }
        }
      }
      __syncthreads();
    }
  }
}

struct radix_cut_t {
  unsigned long long prefix, mask;
};

/// Threshold of the R smallest of n distinct 64-bit keys (n > R): 8-bit radix passes from the top
/// bits, stopping at the first pass whose bucket is taken whole. On return exactly R keys k satisfy
/// (k & mask) <= prefix. hi_at(i) / lo_at(i) give the two 32-bit words of key i; the passes over
/// the high word (the distance) never touch the low one (the id), which only breaks ties. All
/// threads of the block call it.
template <typename HiAt, typename LoAt>
__device__ __forceinline__ radix_cut_t radix_cut(HiAt hi_at, LoAt lo_at, int n, int R, unsigned* hist,
                                                 int* ctrl)
{
  unsigned prefix_hi = 0u, mask_hi = 0u, prefix_lo = 0u, mask_lo = 0u;
  int need = R;
  for (int pass = 0; pass < 8; pass++) {
    const int word = pass < 4 ? 1 : 0, shift = 24 - 8 * (pass & 3);
    for (int i = threadIdx.x; i < 256; i += blockDim.x)
      hist[i] = 0;
    __syncthreads();
    if (word == 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const unsigned h = hi_at(i);
        if ((h & mask_hi) == prefix_hi) atomicAdd(&hist[(h >> shift) & 255], 1u);
      }
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (hi_at(i) != prefix_hi) continue;
        const unsigned l = lo_at(i);
        if ((l & mask_lo) == prefix_lo) atomicAdd(&hist[(l >> shift) & 255], 1u);
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // lane l owns digits 8l .. 8l+7: the digit at which the running count reaches `need`
      const int lane = threadIdx.x;
      unsigned h[8], mine = 0;
#pragma unroll
      for (int t = 0; t < 8; t++) {
        h[t] = hist[8 * lane + t];
        mine += h[t];
      }
      unsigned inc = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
      }
      const unsigned before = inc - mine;
      if (before < static_cast<unsigned>(need) && inc >= static_cast<unsigned>(need)) {
        unsigned cum = before, size = h[7];
        int d        = 7;
#pragma unroll
        for (int t = 0; t < 8; t++) {
          if (cum + h[t] >= static_cast<unsigned>(need)) {
            d    = t;
            size = h[t];
            break;
          }
          cum += h[t];
        }
        ctrl[1] = 8 * lane + d;                  // digit
        ctrl[2] = need - static_cast<int>(cum);  // still needed from that bucket
        ctrl[3] = static_cast<int>(size);        // bucket size
      }
    }
    __syncthreads();
    const int digit = ctrl[1], left = ctrl[2], bucket = ctrl[3];
    if (word == 1) {
      prefix_hi |= static_cast<unsigned>(digit) << shift;
      mask_hi |= 255u << shift;
    } else {
      prefix_lo |= static_cast<unsigned>(digit) << shift;
      mask_lo |= 255u << shift;
    }
    need = left;
    __syncthreads();
    if (bucket == left) break;
  }
  return radix_cut_t{(static_cast<unsigned long long>(prefix_hi) << 32) | prefix_lo,
                     (static_cast<unsigned long long>(mask_hi) << 32) | mask_lo};
}

/// The same threshold as radix_cut with, in the usual case, one counting pass instead of three or
/// four: the high words (distances of one query: a narrow range of bit patterns) are binned over
/// their own range [min, max] into 256 bins, the bin that holds the R-th key is found, and the
/// R-th key itself is ranked among the few members of that bin. Falls back on radix_cut when that
/// bin holds more than 128 keys (many equal or nearly equal distances). hist: 256 words, used as
/// counters and then as the list of the bin's members; ctrl[1], [2], [3], [7] are used.
template <typename HiAt, typename LoAt>
__device__ __forceinline__ radix_cut_t smallest_cut(HiAt hi_at, LoAt lo_at, int n, int R, unsigned* hist,
                                                    int* ctrl)
{
  constexpr int kSide = 128;
  const int lane = threadIdx.x & 31;
  unsigned* uc   = reinterpret_cast<unsigned*>(ctrl);
  for (int i = threadIdx.x; i < 256; i += blockDim.x)
    hist[i] = 0;
  if (threadIdx.x == 0) {
    uc[1] = ~0u;
    uc[2] = 0u;
    uc[7] = 0u;
  }
  __syncthreads();
  unsigned lo = ~0u, hi = 0u;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned h = hi_at(i);
    lo               = min(lo, h);
    hi               = max(hi, h);
  }
  lo = __reduce_min_sync(0xffffffffu, lo);
  hi = __reduce_max_sync(0xffffffffu, hi);
  if (lane == 0) {
    atomicMin(&uc[1], lo);
    atomicMax(&uc[2], hi);
  }
  __syncthreads();
  lo           = uc[1];
  hi           = uc[2];
  const int sh = max(0, 24 - __clz(static_cast<int>(hi - lo)));  // (hi - lo) >> sh < 256
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    atomicAdd(&hist[(hi_at(i) - lo) >> sh], 1u);
  __syncthreads();
  if (threadIdx.x < 32) {
    // lane l owns bins 8l .. 8l+7: the bin at which the running count reaches R
    unsigned h[8], mine = 0;
#pragma unroll
    for (int t = 0; t < 8; t++) {
      h[t] = hist[8 * lane + t];
      mine += h[t];
    }
    unsigned inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned u = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += u;
    }
    const unsigned before = inc - mine;
    if (before < static_cast<unsigned>(R) && inc >= static_cast<unsigned>(R)) {
      unsigned cum = before, size = h[7];
      int d        = 7;
#pragma unroll
      for (int t = 0; t < 8; t++) {
        if (cum + h[t] >= static_cast<unsigned>(R)) {
          d    = t;
          size = h[t];
          break;
        }
        cum += h[t];
      }
      ctrl[1] = 8 * lane + d;               // bin
      ctrl[2] = R - static_cast<int>(cum);  // still needed from that bin
      ctrl[3] = static_cast<int>(size);     // its size
    }
  }
  __syncthreads();
  const unsigned bin = static_cast<unsigned>(ctrl[1]);
  const int left = ctrl[2], bucket = ctrl[3];
  if (bucket == left) {
    // the bin is taken whole: every key whose high word is below the next bin's first value
    unsigned long long top = static_cast<unsigned long long>(lo) + ((static_cast<unsigned long long>(bin) + 1) << sh) - 1;
    if (top > 0xffffffffULL) top = 0xffffffffULL;
    __syncthreads();
    return radix_cut_t{(top << 32) | 0xffffffffULL, ~0ULL};
  }
  if (bucket > kSide) {
    __syncthreads();
    return radix_cut(hi_at, lo_at, n, R, hist, ctrl);
  }
  unsigned long long* side = reinterpret_cast<unsigned long long*>(hist);  // the counters are dead
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned h = hi_at(i);
    if (((h - lo) >> sh) == bin) side[atomicAdd(&uc[7], 1u)] = (static_cast<unsigned long long>(h) << 32) | lo_at(i);
  }
  __syncthreads();
  if (threadIdx.x < bucket) {
    const unsigned long long mine = side[threadIdx.x];
    int below                     = 0;
    for (int j = 0; j < bucket; j++)
      below += side[j] < mine;
    if (below == left - 1) {  // the left-th smallest of the bin is the R-th smallest of all
      uc[2] = static_cast<unsigned>(mine >> 32);
      uc[3] = static_cast<unsigned>(mine);
    }
  }
  __syncthreads();
  const unsigned long long cut = (static_cast<unsigned long long>(uc[2]) << 32) | uc[3];
  __syncthreads();
  return radix_cut_t{cut, ~0ULL};
}

/// Ascending order of cnt <= blockDim.x distinct keys src[0, cnt) into dst (another array): a
/// thread counts the keys below its own and puts it there. No step depends on another, which
/// suits the short lists a merge usually sorts better than a sorting network run by one warp.
__device__ __forceinline__ void rank_sort(const unsigned long long* src, int cnt, unsigned long long* dst)
{
  if (threadIdx.x < cnt) {
    const unsigned long long mine = src[threadIdx.x];
    int below                     = 0;
    for (int j = 0; j < cnt; j++)
      below += src[j] < mine;
    dst[below] = mine;
  }
}

/// float(h) - q for an fp16 bit pattern h: the mixed-precision subtract of sm_100 (PTX ISA 8.6),
/// the same value as converting first (the conversion is exact) without the conversion.
__device__ __forceinline__ float half_minus(unsigned short h, float q)
{
  float d;
  asm("sub.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(h), "f"(q));
  return d;
}

/// Row `id` of an array with `width` elements per row: behind `base`, or (kDealt and a table given)
/// in the memory of the GPU that holds its range (search_kernels.cuh:40-55).
template <bool kDealt, typename T>
__device__ __forceinline__ const T* row_of(const T* base, const row_map& m, int id, int width)
{
  if constexpr (kDealt) {
    if (m.ptrs != nullptr) {
      const int g = id / m.rows;
      return reinterpret_cast<const T*>(m.ptrs[g]) + static_cast<int64_t>(id - g * m.rows) * width;
    }
  }
  return base + static_cast<int64_t>(id) * width;
}

/// Rows that may sit in another GPU's memory are not prefetched into this GPU's L2.
template <bool kDealt>
__device__ __forceinline__ bool may_prefetch(const row_map& m)
{
  return !kDealt || m.ptrs == nullptr;
}

/// The query's side of the sketch distance, made once per query block by its first warp.
/// The reference scores sum_k (c_k s_k - q_k)^2 in fp32 per candidate (search_kernels.cuh:228-251).
/// Expanded: sum_k (c_k s_k)^2 - 2 sum_k c_k (s_k q_k) + sum_k q_k^2. The first sum is a constant
/// of the row, computed when the index is placed (norm [n]); the last is a constant of the
/// query; the middle one becomes an exact integer dot product of the int8 codes with 16-bit weights
/// w_k = rint(s_k q_k / alpha), alpha = max_k |s_k q_k| / 32000 (two codes per dp2a). The value
/// differs from the fp32 sum by the rounding of the weights (at most 1.6e-5 of the largest product
/// per term) and of three fp32 operations. Every operation and its order are stated here and in
/// the CPU checker, which evaluates the same form.
/// Writes w16 [S / 2] (weights of codes 2i and 2i + 1 in the low and high half of word i) and
/// kq[0] = -2 alpha, kq[1] = sum_k q_k^2 (partial sum k mod 32, butterfly with strides 1 .. 16).
__device__ __forceinline__ void sketch_query_setup(const float* __restrict__ qs, const float* __restrict__ scale,
                                                   int S, int* w16, float* kq)
{
  const int lane = threadIdx.x & 31;
  float amax = 0.f, qq = 0.f;
  for (int k = lane; k < S; k += 32) {
    const float q = qs[k];
    amax          = fmaxf(amax, fabsf(__fmul_rn(scale[k], q)));
    qq            = __fmaf_rn(q, q, qq);
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    qq   = __fadd_rn(qq, __shfl_xor_sync(0xffffffffu, qq, o));
  }
  const float alpha = (amax > 0.f && amax <= FLT_MAX) ? __fdiv_rn(amax, 32000.0f) : 1.0f;
  short* w = reinterpret_cast<short*>(w16);
  for (int k = lane; k < S; k += 32) {
    const float r = rintf(__fdiv_rn(__fmul_rn(scale[k], qs[k]), alpha));
    w[k]          = static_cast<short>(r != r ? 0 : static_cast<int>(fminf(fmaxf(r, -32000.0f), 32000.0f)));
  }
  if (lane == 0) {
    kq[0] = -2.0f * alpha;
    kq[1] = qq;
  }
}

/// Sketch distances of the candidates cand[0, n) into dist[0, n): kLw (a power of two >= S / 16)
/// lanes own a row, sixteen codes (one 16-byte load) and their eight weight pairs each; a lane's
/// dot product takes eight dp2a; the lanes of a row add theirs by a butterfly; four rows per lane
/// group are in flight. A lane past the last row works on the last row and a lane past the last
/// chunk on chunk 0 with zero weights; their results are dropped or add 0.
// ---- L2 residency ---------------------------------------------------------------------------------
//
// The int8 sketch and its row constants are the arrays every query reads most often (hundreds of
// rows per round) and, for an index of a million rows, small enough to stay in the 126 MB L2 cache
// next to everything else; the fp16 vectors, the lists and the neighbor table are read once or a
// few times per batch and are many times larger. When the host finds that the sketch fits, the
// kernels load sketch rows and constants with an evict-last policy and the large arrays with an
// evict-first policy, so that the streaming reads do not push the sketch out.

__device__ __forceinline__ unsigned long long l2_policy_keep()
{
  unsigned long long p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ unsigned long long l2_policy_stream()
{
  unsigned long long p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ uint4 ldg16_hint(const void* a, unsigned long long policy)
{
  uint4 v;
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(a), "l"(policy));
  return v;
}

__device__ __forceinline__ float ldg_f32_hint(const float* a, unsigned long long policy)
{
  float v;
  asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(a), "l"(policy));
  return v;
}

__device__ __forceinline__ int ldg_i32_hint(const int* a, unsigned long long policy)
{
  int v;
  asm volatile("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(a), "l"(policy));
  return v;
}

template <int kLw, bool kDealt>
__device__ __forceinline__ void sketch_rows_int(const int* cand, int n, const signed char* __restrict__ sketch,
                                                const float* __restrict__ norm, const row_map& map, int S,
                                                const int* w16, const float* kq, float* dist, bool keep)
{
  constexpr int kG = 32 / kLw;  // rows per warp and step
  constexpr int kU = 4;          // rows of a lane group in flight
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int sub = lane % kLw, grp = lane / kLw;
  const bool live  = 16 * sub < S;
  const int subc   = live ? sub : 0;
  int w[8];
  {
    const int4 w0 = reinterpret_cast<const int4*>(w16)[2 * subc];
    const int4 w1 = reinterpret_cast<const int4*>(w16)[2 * subc + 1];
    w[0] = w0.x, w[1] = w0.y, w[2] = w0.z, w[3] = w0.w, w[4] = w1.x, w[5] = w1.y, w[6] = w1.z, w[7] = w1.w;
#pragma unroll
    for (int b = 0; b < 8; b++)
      if (!live) w[b] = 0;
  }
  const float beta = kq[0], qq = kq[1];
  const unsigned long long pol = l2_policy_keep();
  const int rpp = nw * kG;  // rows per step of the block
  for (int jb = 0; jb < n; jb += kU * rpp) {
    uint4 c[kU];
    float nrm[kU];
    int j[kU];
#pragma unroll
    for (int u = 0; u < kU; u++) {
      j[u]            = jb + u * rpp + warp * kG + grp;
      const int id    = cand[min(j[u], n - 1)];
      const uint4* row = reinterpret_cast<const uint4*>(row_of<kDealt>(sketch, map, id, S)) + subc;
      if (keep) {
        c[u]   = ldg16_hint(row, pol);
        nrm[u] = ldg_f32_hint(norm + id, pol);
      } else {
        c[u]   = __ldg(row);
        nrm[u] = __ldg(norm + id);
      }
    }
#pragma unroll
    for (int u = 0; u < kU; u++) {
      int d = __dp2a_lo(w[0], static_cast<int>(c[u].x), 0);
      d     = __dp2a_hi(w[1], static_cast<int>(c[u].x), d);
      d     = __dp2a_lo(w[2], static_cast<int>(c[u].y), d);
      d     = __dp2a_hi(w[3], static_cast<int>(c[u].y), d);
      d     = __dp2a_lo(w[4], static_cast<int>(c[u].z), d);
      d     = __dp2a_hi(w[5], static_cast<int>(c[u].z), d);
      d     = __dp2a_lo(w[6], static_cast<int>(c[u].w), d);
      d     = __dp2a_hi(w[7], static_cast<int>(c[u].w), d);
#pragma unroll
      for (int o = 1; o < kLw; o <<= 1)
        d += __shfl_xor_sync(0xffffffffu, d, o);
      if (j[u] < n && sub == 0)
        dist[j[u]] = fmaxf(__fadd_rn(nrm[u], __fmaf_rn(beta, static_cast<float>(d), qq)), 0.f);
    }
  }
}

/// Eight int8 codes (two 32-bit words) against eight (scale, query) pairs: sum of
/// (code * scale - q)^2 with two fused multiply-adds per code, in code order. The int8 -> float
/// conversion: one byte permute makes the fp16 patterns 0x64bb = 1024 + (code + 128) of two codes,
/// and the mixed-precision subtract of 1152 gives each code exactly, off the conversion pipe.
__device__ __forceinline__ float sketch_chunk8(unsigned w0, unsigned w1, const float* s, const float* q)
{
  const unsigned x0 = w0 ^ 0x80808080u, x1 = w1 ^ 0x80808080u;  // code + 128 in every byte
  float d           = 0.f;
#pragma unroll
  for (int p = 0; p < 4; p++) {
    const unsigned hh = __byte_perm(p < 2 ? x0 : x1, 0x64646464u, (p & 1) ? 0x4342 : 0x4140);
    const float c0    = half_minus(static_cast<unsigned short>(hh & 0xffffu), 1152.0f);
    const float c1    = half_minus(static_cast<unsigned short>(hh >> 16), 1152.0f);
    const float t0    = __fmaf_rn(c0, s[2 * p], -q[2 * p]);
    d                 = __fmaf_rn(t0, t0, d);
    const float t1    = __fmaf_rn(c1, s[2 * p + 1], -q[2 * p + 1]);
    d                 = __fmaf_rn(t1, t1, d);
  }
  return d;
}

/// The sketch distance in the reference's own fp32 terms, sum_k (c_k s_k - q_k)^2
/// (search_kernels.cuh:228-251), for the waves: there a candidate's row arrives from memory later
/// than the arithmetic on it takes, so the form that needs nothing but the row (no row constant)
/// is the faster one; the first round, whose rows are mostly in the L2 cache already, is bound by
/// instructions and takes the integer form above. Summation order (shared with the CPU checker):
/// chunk c of 8 codes is partial sum c (two fused multiply-adds per code, in code order), a
/// butterfly over the next power of two >= S / 8 partial sums with strides 1, 2, 4, ... A lane
/// holds two neighbouring chunks (one 16-byte load) and adds them itself (stride 1); kLw (a power
/// of two >= S / 16) lanes own a row; two rows per lane group are in flight. A lane past the last
/// chunk works on chunk 0 with scales and query 0 and adds exactly 0.
template <int kLw, bool kDealt>
__device__ __forceinline__ void sketch_rows_f32(const int* cand, int n, const signed char* __restrict__ sketch,
                                                const row_map& map, int S, const float* sc, const float* qv,
                                                float* dist)
{
  constexpr int kG = 32 / kLw;  // rows per warp and step
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int sub = lane % kLw, grp = lane / kLw;
  const bool live = 16 * sub < S;
  const int subc  = live ? sub : 0;
  // the lane's sixteen scales and query values, 16 bytes at a time (both arrays start on 16-byte
  // boundaries): a quarter of the shared-memory traffic of single words
  float cs[16], cq[16];
#pragma unroll
  for (int b = 0; b < 4; b++) {
    const float4 s4 = live ? reinterpret_cast<const float4*>(sc + sub * 16)[b] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 q4 = live ? reinterpret_cast<const float4*>(qv + sub * 16)[b] : make_float4(0.f, 0.f, 0.f, 0.f);
    cs[4 * b] = s4.x, cs[4 * b + 1] = s4.y, cs[4 * b + 2] = s4.z, cs[4 * b + 3] = s4.w;
    cq[4 * b] = q4.x, cq[4 * b + 1] = q4.y, cq[4 * b + 2] = q4.z, cq[4 * b + 3] = q4.w;
  }
  const int rpp = nw * kG;  // rows per step of the block
  for (int jb = 0; jb < n; jb += 2 * rpp) {
    uint4 w[2];
    int j[2];
#pragma unroll
    for (int u = 0; u < 2; u++) {
      j[u]         = jb + u * rpp + warp * kG + grp;
      const int id = cand[min(j[u], n - 1)];
      w[u] = __ldg(reinterpret_cast<const uint4*>(row_of<kDealt>(sketch, map, id, S)) + subc);
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const float d0 = sketch_chunk8(w[u].x, w[u].y, cs, cq);
      const float d1 = sketch_chunk8(w[u].z, w[u].w, cs + 8, cq + 8);
      float d        = __fadd_rn(d0, d1);
#pragma unroll
      for (int o = 1; o < kLw; o <<= 1)
        d = __fadd_rn(d, __shfl_xor_sync(0xffffffffu, d, o));
      if (j[u] < n && sub == 0) dist[j[u]] = d;
    }
  }
}

/// Where element i of the query sits in shared memory for exact_pair: within every step of 64
/// elements the 16-byte chunks are dealt so that the eight lanes of a row group read consecutive
/// chunks with each of their two loads (chunks 0, 2, 4, ... first, then 1, 3, 5, ...): one
/// wavefront per load instead of two. The array takes the dimension rounded up to 64 floats.
__device__ __forceinline__ int query_slot(int i)
{
  const int chunk = (i & 63) >> 2;
  return (i & ~63) + ((((chunk & 1) << 3) + (chunk >> 1)) << 2) + (i & 3);
}

/// Rows j and j + stride of a lane group: squared distances of two fp16 rows to the query fq (laid
/// out by query_slot)
/// (shared memory, read 16 bytes at a time).
/// Both row pointers are valid (a row that is not wanted is replaced by any row by the caller, who
/// drops the result). kMode 0: any D that is a multiple of 8; 1: D a multiple of 128, so no step
/// needs a bounds check; 2: D = 128, one step with constant offsets.
template <int kMode>
__device__ __forceinline__ void exact_pair(const uint4* const (&row)[2], int Drt, int sub, const float* fq,
                                           float (&out)[2])
{
  constexpr bool kWhole = kMode != 0;
  const int D           = kMode == 2 ? 128 : Drt;
  float acc[2][4];
#pragma unroll
  for (int u = 0; u < 2; u++)
#pragma unroll
    for (int t = 0; t < 4; t++)
      acc[u][t] = 0.f;
  // two 16-byte steps of both rows are loaded before any of them is used
  for (int h0 = 8 * sub; h0 < D; h0 += 128) {
    uint4 v[2][2];
#pragma unroll
    for (int s = 0; s < 2; s++)
#pragma unroll
      for (int u = 0; u < 2; u++)
        if (kWhole || h0 + 64 * s < D) v[s][u] = __ldg(row[u] + ((h0 + 64 * s) >> 3));
#pragma unroll
    for (int s = 0; s < 2; s++) {
      const int hs = h0 + 64 * s;
      if (kWhole || hs < D) {
        const float4 q0 = *reinterpret_cast<const float4*>(fq + (hs - 8 * sub) + 4 * sub);
        const float4 q1 = *reinterpret_cast<const float4*>(fq + (hs - 8 * sub) + 4 * sub + 32);
        const float qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const unsigned h2[4] = {v[s][u].x, v[s][u].y, v[s][u].z, v[s][u].w};
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const float a = half_minus(static_cast<unsigned short>(h2[t] & 0xffffu), qq[2 * t]);
            const float b = half_minus(static_cast<unsigned short>(h2[t] >> 16), qq[2 * t + 1]);
            acc[u][t]     = __fmaf_rn(b, b, __fmaf_rn(a, a, acc[u][t]));
          }
        }
      }
    }
  }
  // butterfly over the 32 partial sums, strides 1, 2 (inside the lane), then 4, 8, 16 (lanes)
#pragma unroll
  for (int u = 0; u < 2; u++) {
    float v = __fadd_rn(__fadd_rn(acc[u][0], acc[u][1]), __fadd_rn(acc[u][2], acc[u][3]));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1)
      v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    out[u] = v;
  }
}

/// Squared distances of the fp16 rows sid[0, ns) (entries < 0 are skipped) to the fp32 query fq,
/// written over sdv. Summation order (shared with the CPU checker): element pair k feeds partial
/// sum k mod 32 with two fused multiply-adds; a butterfly over the 32 partial sums with strides
/// 1, 2, 4, 8, 16 (search_kernels.cuh:325-342 is the reference's warp-per-row form of the same
/// sum). Eight lanes own a row, each reading 16 bytes per step (partial sums 4 lane .. 4 lane + 3);
/// a warp works on eight rows at a time.
template <bool kDealt, int kMode>
__device__ __forceinline__ void exact_rows(const int* sid, int ns, const __half* __restrict__ vectors,
                                           const row_map& map, int Drt, const float* fq, float* sdv)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int sub = lane & 7, grp = lane >> 3;
  const int D   = kMode == 2 ? 128 : Drt;
  for (int jb = warp * 4 + grp; jb < ns + warp * 4 + grp; jb += nw * 8) {
    int j[2];
    bool wanted[2];
    const uint4* row[2];
#pragma unroll
    for (int u = 0; u < 2; u++) {
      j[u]         = jb + u * nw * 4;
      const int id = j[u] < ns ? sid[j[u]] : -1;
      wanted[u]    = id >= 0;
      // a slot without a row works on a row this GPU holds (cached after its first use) and drops
      // the result
      row[u] = reinterpret_cast<const uint4*>(row_of<kDealt>(vectors, map, wanted[u] ? id : map.local, D));
    }
    float out[2];
    exact_pair<kMode>(row, D, sub, fq, out);
#pragma unroll
    for (int u = 0; u < 2; u++)
      if (wanted[u] && sub == 0) sdv[j[u]] = out[u];
  }
}

template <bool kDealt>
__device__ __forceinline__ void exact_distances(const int* sid, int ns, const __half* __restrict__ vectors,
                                                const row_map& map, int D, const float* fq, float* sdv)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (D == 128) {
    exact_rows<kDealt, 2>(sid, ns, vectors, map, D, fq, sdv);
  } else if ((D & 127) == 0) {
    exact_rows<kDealt, 1>(sid, ns, vectors, map, D, fq, sdv);
  } else if ((D & 7) == 0) {
    exact_rows<kDealt, 0>(sid, ns, vectors, map, D, fq, sdv);
  } else {
    for (int j = warp; j < ns; j += nw) {
      if (sid[j] < 0) continue;
      const __half2* row = reinterpret_cast<const __half2*>(row_of<kDealt>(vectors, map, sid[j], D));
      float acc          = 0.f;
      for (int k = lane; k < D / 2; k += 32) {
        const float2 x = __half22float2(row[k]);
        const float a  = __fsub_rn(x.x, fq[2 * k]);
        const float b  = __fsub_rn(x.y, fq[2 * k + 1]);
        acc            = __fmaf_rn(b, b, __fmaf_rn(a, a, acc));
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1)
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
      if (lane == 0) sdv[j] = acc;
    }
  }
  __syncthreads();
}

/// Merge the new (distance, id) pairs sid / sdv [0, ns) (entries with sid < 0 are skipped; no id is
/// in the kept list already) into the kept list of KO: the KO smallest keys, ascending, padded
/// with (-1, +inf), written to pb / pd. Same result as sorting kept + new and taking the first KO
/// distinct keys (search_kernels.cuh:372-415). A new key beyond the last entry of a full kept list
/// cannot make it and is dropped at once; what remains is sorted directly when it is short, or the
/// KO smallest are cut out by radix passes first. kid / kd: the kept list as it was (shared
/// memory), null when it starts empty. pool holds KO + ns keys, sorted holds 2 * P (P a power of
/// two >= KO).
__device__ __forceinline__ void merge_into_kept(unsigned long long* pool,
                                                unsigned long long* sorted,
                                                int P,
                                                long long* pb,
                                                float* pd,
                                                int KO,
                                                const int* kid,
                                                const float* kd,
                                                const int* sid,
                                                const float* sdv,
                                                int ns,
                                                unsigned* hist,
                                                int* ctrl)
{
  const bool fresh = kid == nullptr;
  if (threadIdx.x == 0) ctrl[6] = 0;
  // the kept list is packed (valid entries first): nk = first index without an id
  int nk = 0;
  if (!fresh) {
    int lo = 0, hi = KO;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (kid[mid] >= 0)
        lo = mid + 1;
      else
        hi = mid;
    }
    nk = lo;
  }
  const unsigned long long bound =
    nk == KO && KO > 0 ? rank_key(kd[KO - 1], static_cast<unsigned>(kid[KO - 1])) : kNoKey;
  __syncthreads();
  for (int i = threadIdx.x; i < nk; i += blockDim.x)
    pool[i] = rank_key(kd[i], static_cast<unsigned>(kid[i]));
  for (int i = threadIdx.x; i < ns; i += blockDim.x) {
    if (sid[i] < 0) continue;
    const unsigned long long k = rank_key(sdv[i], static_cast<unsigned>(sid[i]));
    if (k < bound) pool[nk + atomicAdd(&ctrl[6], 1)] = k;
  }
  __syncthreads();
  const int total = nk + ctrl[6];
  int cnt         = min(total, KO);
  constexpr int kRankMax = 128;  // keys sorted by ranking, one thread per key (blocks have >= 128 threads)
  if (total <= 2 * P) {
    if (total <= kRankMax) {
      rank_sort(pool, total, sorted);
    } else {
      int width = P;
      while (width < total)
        width <<= 1;
      for (int i = threadIdx.x; i < width; i += blockDim.x)
        sorted[i] = i < total ? pool[i] : kNoKey;
      __syncthreads();
      bitonic_sort(sorted, width);
    }
  } else {
    // the KO smallest are cut out first (into the upper half of the sort region), then sorted
    unsigned long long* picked = sorted + max(P, 32);
    auto hi_at          = [&](int i) { return static_cast<unsigned>(pool[i] >> 32); };
    auto lo_at          = [&](int i) { return static_cast<unsigned>(pool[i]); };
    const radix_cut_t c = smallest_cut(hi_at, lo_at, total, KO, hist, ctrl);
    if (threadIdx.x == 0) ctrl[0] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const unsigned long long k = pool[i];
      if ((k & c.mask) <= c.prefix) {
        const int s = atomicAdd(&ctrl[0], 1);
        if (s < P) picked[s] = k;
      }
    }
    __syncthreads();
    if (KO <= kRankMax) {
      rank_sort(picked, KO, sorted);
    } else {
      for (int i = threadIdx.x; i < P; i += blockDim.x)
        sorted[i] = i < KO ? picked[i] : kNoKey;
      __syncthreads();
      bitonic_sort(sorted, P);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < KO; i += blockDim.x) {
    const unsigned long long k = i < cnt ? sorted[i] : kNoKey;
    pb[i] = k == kNoKey ? -1 : static_cast<long long>(static_cast<unsigned>(k & 0xffffffffULL));
    pd[i] = k == kNoKey ? INFINITY : __uint_as_float(static_cast<unsigned>(k >> 32));
  }
}


// kThreads: 128 with eight blocks per multiprocessor when a block's shared memory allows that; a
// round whose hash set is too large for eight blocks runs 256 or 512 threads per block instead, so
// that the blocks that do fit still bring 32 warps to a multiprocessor.
template <bool kRows, bool kDealt, int kThreads>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) round_kernel(const round_args a)
{
  extern __shared__ __align__(16) int smem[];
  const round_layout lay(a);
  const int q = blockIdx.x;
  int* table  = smem + lay.table;
  int* cand   = a.cand_global ? a.cand_global + static_cast<int64_t>(q) * a.nmax : smem + lay.cand;
  float* dist = a.dist_global ? a.dist_global + static_cast<int64_t>(q) * a.nmax
                              : reinterpret_cast<float*>(smem + lay.dist);
  unsigned long long* pool   = reinterpret_cast<unsigned long long*>(smem + lay.pool);
  unsigned long long* sorted = reinterpret_cast<unsigned long long*>(smem + lay.sorted);
  int* sid                   = smem + lay.sid;
  float* sdv                 = reinterpret_cast<float*>(smem + lay.sdv);
  int* w16                   = smem + lay.qv;
  float* kq                  = reinterpret_cast<float*>(smem + lay.sc);
  float* fq                  = reinterpret_cast<float*>(smem + lay.fq);
  int* st                    = smem + lay.st;
  int* len                   = smem + lay.len;
  unsigned* hist             = reinterpret_cast<unsigned*>(smem + lay.hist);
  int* wsum                  = smem + lay.wsum;
  int* ctrl                  = smem + lay.ctrl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int S    = a.sw;
  long long* pb  = a.si + static_cast<int64_t>(q) * a.KO;
  float* pd      = a.sd + static_cast<int64_t>(q) * a.KO;
  const bool fresh = a.fresh != 0;

  // The integer form of the sketch distance serves the first round of a search that reranks
  // exactly. Waves take the fp32 sum (see sketch_rows_f32), and so does every round of a search
  // that ranks by sketch distance: there the distances of all rounds meet in one kept list, where
  // an id found twice must bring the same key both times.
  const bool int_form = !kRows && !a.sketch_rank;
  if (int_form) {
    if (warp == 0) sketch_query_setup(a.qs + static_cast<int64_t>(q) * S, a.scale, S, w16, kq);
  } else {
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
      reinterpret_cast<float*>(w16)[i] = a.qs[static_cast<int64_t>(q) * S + i];
      kq[i]                            = a.scale[i];
    }
  }
  if (!a.sketch_rank)
    for (int i = threadIdx.x; i < a.D; i += blockDim.x)
      fq[(a.D & 7) ? i : query_slot(i)] = a.Q[static_cast<int64_t>(q) * a.D + i];
  if (threadIdx.x == 0) ctrl[4] = 0;  // distinct ids
  // the kept list as the round finds it: read once, used by the start points, by the filter of
  // already kept ids and by the merge
  int* kid  = smem + lay.kid;
  float* kd = reinterpret_cast<float*>(smem + lay.kd);
  if (!fresh)
    for (int i = threadIdx.x; i < a.KO; i += blockDim.x) {
      kid[i] = static_cast<int>(pb[i]);
      kd[i]  = pd[i];
    }

  // cycles per phase of this block (observation only): start points / segments, gather, sketch
  // scoring, selection, filter + prefetch, exact distances, merge
  long long t_prev = 0;
  auto tick = [&](int i) {
    if (a.phase != nullptr && threadIdx.x == 0) {
      const long long t = clock64();
      if (i >= 0) a.phase[static_cast<int64_t>(q) * 8 + i] += t - t_prev;
      t_prev = t;
    }
  };
  tick(-1);
  int total = 0, nseg = a.nseg;
  if constexpr (kRows) {
    // start points: the first nseg kept entries that no earlier wave expanded
    // (search_kernels.cuh:571-631); earlier start points go through a hash set in the table region
    int* pdone = a.done + static_cast<int64_t>(q) * a.done_stride;
    for (int i = threadIdx.x; i < a.pick_slots; i += blockDim.x)
      table[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < a.done_off; i += blockDim.x) {
      const int v = pdone[i];
      if (v < 0) continue;
      unsigned h = (static_cast<unsigned>(v) * kIdHash) & (a.pick_slots - 1);
      for (int p = 0; p < a.pick_slots; p++) {
        const int prev = atomicCAS(&table[h], -1, v);
        if (prev == -1 || prev == v) break;
        h = (h + 1) & (a.pick_slots - 1);
      }
    }
    __syncthreads();
    const int per       = (a.KO + kThreads - 1) / kThreads;
    const int i0        = threadIdx.x * per;
    unsigned fresh_bits = 0;
    int mine            = 0;
    for (int i = i0; i < min(a.KO, i0 + per); i++) {
      const int v = kid[i];
      bool f      = v >= 0;
      if (f) {
        unsigned h = (static_cast<unsigned>(v) * kIdHash) & (a.pick_slots - 1);
        for (int p = 0; p < a.pick_slots; p++) {
          const int t = table[h];
          if (t == -1) break;
          if (t == v) {
            f = false;
            break;
          }
          h = (h + 1) & (a.pick_slots - 1);
        }
      }
      if (f) {
        fresh_bits |= 1u << (i - i0);
        mine++;
      }
    }
    int nfresh = 0;
    int at     = block_scan<kThreads>(mine, wsum, nfresh);
    for (int i = i0; i < min(a.KO, i0 + per); i++)
      if (fresh_bits & (1u << (i - i0))) {
        if (at < a.nseg) {
          const int v            = kid[i];
          st[at]                 = v;
          pdone[a.done_off + at] = v;
          // its table row is read next: start bringing it into L2
          if (may_prefetch<kDealt>(a.table_map)) {
            const char* row = reinterpret_cast<const char*>(a.table + static_cast<int64_t>(v) * a.table_len);
            for (int b = 0; b < a.table_len * 4; b += 128)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(row + b));
          }
        }
        at++;
      }
    nseg = min(nfresh, a.nseg);
    for (int o = nseg + threadIdx.x; o < a.nseg; o += blockDim.x)
      pdone[a.done_off + o] = -1;
    total = nseg * a.table_len;
    if (threadIdx.x == 0) ctrl[5] = nseg;
    __syncthreads();
  } else {
    // segment starts and lengths; every segment is either empty or `read` entries long
    int mine = 0;
    for (int c = threadIdx.x; c < a.nseg; c += blockDim.x) {
      const int2 sl = a.seg[static_cast<int64_t>(q) * a.nseg + c];
      st[c]         = sl.x;
      len[c]        = sl.y;
      mine += sl.y;
      if (sl.y > 0) {  // the run of list entries is read next: start bringing it into L2
        const char* run = reinterpret_cast<const char*>(a.lists + static_cast<int64_t>(c) * a.stride + sl.x);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(run));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(run + sl.y * 4 - 4));
      }
    }
    block_scan<kThreads>(mine, wsum, total);
  }

  // distinct ids through an open-addressing hash set (search_kernels.cuh:191-225); a group of lps
  // threads walks one segment, so consecutive threads read consecutive entries, and every thread
  // has four segments' loads in flight before it touches the set
  tick(0);
  const int HT = hash_slots_of(total, a.cap_slots, a.hash_twelfths);
  for (int i = threadIdx.x; i < HT / 4; i += blockDim.x)
    reinterpret_cast<int4*>(table)[i] = make_int4(-1, -1, -1, -1);
  __syncthreads();
  {
    const int maxlen = kRows ? a.table_len : a.lr;
    int lps          = 1;
    while (lps < maxlen && lps < kThreads)
      lps <<= 1;
    const int within0 = threadIdx.x & (lps - 1);
    const int spp     = kThreads / lps;  // segments per pass
    const int seg0    = threadIdx.x / lps;
    // the large arrays pass through the L2 cache without staying when the sketch is to be kept there
    const bool stream = a.keep_sketch != 0 && (!kDealt || !kRows || a.table_map.ptrs == nullptr);
    const unsigned long long spol = l2_policy_stream();
    // loop bounds are the same for every thread: the slot counter below is updated once per warp
    for (int wb = 0; wb < maxlen; wb += lps) {
      const int w0 = wb + within0;
      for (int sb = 0; sb < nseg; sb += 4 * spp) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int s = sb + seg0 + u * spp;
          v[u]        = -1;
          if (s < nseg && w0 < maxlen) {
            if constexpr (kRows) {
              const int* at = row_of<kDealt>(a.table, a.table_map, st[s], a.table_len) + w0;
              v[u]          = stream ? ldg_i32_hint(at, spol) : __ldg(at);
            } else {
              const int* at = a.lists + static_cast<int64_t>(s) * a.stride + st[s] + w0;
              if (w0 < len[s]) v[u] = stream ? ldg_i32_hint(at, spol) : __ldg(at);
            }
          }
        }
        int mine = 0;
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int id = v[u];
          bool is_new  = false;
          if (id >= 0) {  // else nothing read, or the padding of a table row
            unsigned s = home_slot(id, HT);
            for (int p = 0; p < HT; p++) {
              const int prev = atomicCAS(&table[s], -1, id);
              if (prev == -1) {
                is_new = true;
                break;
              }
              if (prev == id) break;
              s = s + 1 == static_cast<unsigned>(HT) ? 0u : s + 1;
            }
          }
          if (!is_new) v[u] = -1;
          mine += is_new;
        }
        // slots for the new ids of the whole warp with one update of the counter
        __syncwarp();
        int inc = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += up;
        }
        int base = 0;
        if (lane == 31 && inc > 0) base = atomicAdd(&ctrl[4], inc);
        base   = __shfl_sync(0xffffffffu, base, 31);
        int at = base + inc - mine;
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (v[u] >= 0) {
            if (at < a.nmax) cand[at] = v[u];
            at++;
          }
      }
    }
  }
  __syncthreads();
  const int n = min(ctrl[4], a.nmax);
  tick(1);

  // int8 sketch distances (search_kernels.cuh:228-251), sixteen codes per lane, S / 16 lanes
  // (rounded up to a power of two) per row
  if (!int_form) {
    const float* qv = reinterpret_cast<const float*>(w16);
    if (S <= 16) {
      sketch_rows_f32<1, kDealt>(cand, n, a.sketch, a.sketch_map, S, kq, qv, dist);
    } else if (S <= 32) {
      sketch_rows_f32<2, kDealt>(cand, n, a.sketch, a.sketch_map, S, kq, qv, dist);
    } else if (S <= 64) {
      sketch_rows_f32<4, kDealt>(cand, n, a.sketch, a.sketch_map, S, kq, qv, dist);
    } else if (S <= 128) {
      sketch_rows_f32<8, kDealt>(cand, n, a.sketch, a.sketch_map, S, kq, qv, dist);
    } else if (S <= 256) {
      sketch_rows_f32<16, kDealt>(cand, n, a.sketch, a.sketch_map, S, kq, qv, dist);
    } else {
      sketch_rows_f32<32, kDealt>(cand, n, a.sketch, a.sketch_map, S, kq, qv, dist);
    }
  } else {
    const bool keep = a.keep_sketch != 0 && may_prefetch<kDealt>(a.sketch_map);
    if (S <= 16) {
      sketch_rows_int<1, kDealt>(cand, n, a.sketch, a.sketch_norm, a.sketch_map, S, w16, kq, dist, keep);
    } else if (S <= 32) {
      sketch_rows_int<2, kDealt>(cand, n, a.sketch, a.sketch_norm, a.sketch_map, S, w16, kq, dist, keep);
    } else if (S <= 64) {
      sketch_rows_int<4, kDealt>(cand, n, a.sketch, a.sketch_norm, a.sketch_map, S, w16, kq, dist, keep);
    } else if (S <= 128) {
      sketch_rows_int<8, kDealt>(cand, n, a.sketch, a.sketch_norm, a.sketch_map, S, w16, kq, dist, keep);
    } else if (S <= 256) {
      sketch_rows_int<16, kDealt>(cand, n, a.sketch, a.sketch_norm, a.sketch_map, S, w16, kq, dist, keep);
    } else {
      sketch_rows_int<32, kDealt>(cand, n, a.sketch, a.sketch_norm, a.sketch_map, S, w16, kq, dist, keep);
    }
  }
  __syncthreads();
  tick(2);
  if (a.tap_cand != nullptr) {
    for (int i = threadIdx.x; i < min(n, a.tap_cap); i += blockDim.x) {
      a.tap_cand[static_cast<int64_t>(q) * a.tap_cap + i] = cand[i];
      a.tap_dist[static_cast<int64_t>(q) * a.tap_cap + i] = dist[i];
    }
    if (threadIdx.x == 0) a.tap_n[q] = n;
  }

  // the nearest by (sketch distance, id) (search_kernels.cuh:259-322 takes equal distances at the
  // cut in any order)
  const int R = a.sketch_rank ? a.KO : a.R;
  int ns      = n;
  if (n > R) {
    auto key_at = [&](int i) { return rank_key(dist[i], static_cast<unsigned>(cand[i])); };
    auto hi_at          = [&](int i) { return __float_as_uint(dist[i]); };
    auto lo_at          = [&](int i) { return static_cast<unsigned>(cand[i]); };
    const radix_cut_t c = smallest_cut(hi_at, lo_at, n, R, hist, ctrl);
    if (threadIdx.x == 0) ctrl[0] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      if ((key_at(i) & c.mask) <= c.prefix) {
        const int s = atomicAdd(&ctrl[0], 1);
        if (s < R) {
          sid[s] = cand[i];
          sdv[s] = dist[i];
        }
      }
    }
    ns = R;
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      sid[i] = cand[i];
      sdv[i] = dist[i];
    }
  }
  __syncthreads();

  tick(3);
  // a selected id that is already in the kept list brings the key it already has there: drop it
  // before the vectors are read (the reference reranks it again and collapses the equal keys)
  if (!fresh) {
    int HK = 64;
    while (HK < 2 * a.KO)
      HK <<= 1;
    for (int i = threadIdx.x; i < HK; i += blockDim.x)
      table[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < a.KO; i += blockDim.x) {
      const int v = kid[i];
      if (v < 0) continue;
      unsigned h = (static_cast<unsigned>(v) * kIdHash) & (HK - 1);
      for (int p = 0; p < HK; p++) {
        const int prev = atomicCAS(&table[h], -1, v);
        if (prev == -1 || prev == v) break;
        h = (h + 1) & (HK - 1);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ns; i += blockDim.x) {
      const int v = sid[i];
      unsigned h  = (static_cast<unsigned>(v) * kIdHash) & (HK - 1);
      for (int p = 0; p < HK; p++) {
        const int t = table[h];
        if (t == -1) break;
        if (t == v) {
          sid[i] = -1;
          break;
        }
        h = (h + 1) & (HK - 1);
      }
    }
    __syncthreads();
  }
  int reranked = 0;
  if (!a.sketch_rank) {
    // every row about to be read is asked for at once (128-byte lines into L2), so the distance
    // loop below finds most of them on the way
    const int row_bytes = a.D * 2;
    for (int r = threadIdx.x; r < (may_prefetch<kDealt>(a.vector_map) ? ns : 0); r += blockDim.x) {
      if (sid[r] < 0) continue;
      const char* row = reinterpret_cast<const char*>(a.vectors + static_cast<int64_t>(sid[r]) * a.D);
      for (int b = 0; b < row_bytes; b += 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(row + b));
    }
    if (a.stats != nullptr) {
      int mine = 0;
      for (int i = threadIdx.x; i < ns; i += blockDim.x)
        mine += sid[i] >= 0;
      block_scan<kThreads>(mine, wsum, reranked);
    }
    tick(4);
    exact_distances<kDealt>(sid, ns, a.vectors, a.vector_map, a.D, fq, sdv);
    tick(5);
  }
  merge_into_kept(pool, sorted, a.P, pb, pd, a.KO, fresh ? nullptr : kid, kd, sid, sdv, ns, hist, ctrl);
  __syncthreads();
  tick(6);
  if (a.stats != nullptr && threadIdx.x == 0) {
    long long* s = a.stats + static_cast<int64_t>(q) * 8;
    if constexpr (kRows) {
      s[4] += ctrl[5];
      s[5] += n;
    } else {
      s[2] += total;
      s[3] += n;
    }
    if (!a.sketch_rank) s[6] += ns;  // rows the reference reranks
    s[7] += reranked;  // rows read here (those already kept are skipped)
  }
}

// search_kernels.cuh:634-669: exact distances of the first R kept entries, best k of them.
__global__ void __launch_bounds__(kRoundThreads) final_rerank_kernel(const long long* __restrict__ si,
                                                                     int KO,
                                                                     int R,
                                                                     const __half* __restrict__ vectors,
                                                                     const row_map vector_map,
                                                                     int D,
                                                                     const float* __restrict__ Q,
                                                                     int k,
                                                                     int P,
                                                                     long long* __restrict__ bi,
                                                                     float* __restrict__ bd,
                                                                     long long* __restrict__ stats)
{
  extern __shared__ __align__(16) int smem[];
  unsigned long long* pool   = reinterpret_cast<unsigned long long*>(smem);  // [k + R]
  unsigned long long* sorted = pool + ((k + R + 1) & ~1);                    // [P]
  int* sid                   = reinterpret_cast<int*>(sorted + max(2 * P, 64));  // sorted [max(2 P, 64)]; sid [R]
  float* sdv                 = reinterpret_cast<float*>(sid + ((R + 3) & ~3));
  float* fq                  = sdv + ((R + 3) & ~3);                         // [D]
  unsigned* hist             = reinterpret_cast<unsigned*>(fq + ((D + 63) & ~63));
  int* wsum                  = reinterpret_cast<int*>(hist + 256);
  int* ctrl                  = wsum + 16;
  const int q                = blockIdx.x;
  const long long* ps        = si + static_cast<int64_t>(q) * KO;
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    fq[(D & 7) ? i : query_slot(i)] = Q[static_cast<int64_t>(q) * D + i];
  // the kept list is packed (valid entries first), so the valid ones among the first R are a prefix
  int mine = 0;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const long long v = ps[i];
    sid[i]            = static_cast<int>(v);
    if (v >= 0) mine++;
  }
  int ns = 0;
  block_scan(mine, wsum, ns);
  exact_distances<true>(sid, ns, vectors, vector_map, D, fq, sdv);
  merge_into_kept(pool, sorted, P, bi + static_cast<int64_t>(q) * k, bd + static_cast<int64_t>(q) * k,
                  k, nullptr, nullptr, sid, sdv, ns, hist, ctrl);
  if (stats != nullptr && threadIdx.x == 0) {
    stats[static_cast<int64_t>(q) * 8 + 6] += ns;
    stats[static_cast<int64_t>(q) * 8 + 7] += ns;
  }
}

// search_kernels.cuh:517-564: kept lists of nsrc sources -> the nearest copy of each id -> best
// KO. The sources are rows of arrays in this GPU's own memory (the exchange brought them here).
__global__ void merge_kept_kernel(const long long* __restrict__ src_i,
                                  const float* __restrict__ src_d,
                                  int nsrc,
                                  int64_t src_stride,
                                  int KO,
                                  int P,
                                  long long* __restrict__ si,
                                  float* __restrict__ sd)
{
  extern __shared__ __align__(16) int smem[];
  unsigned long long* mk = reinterpret_cast<unsigned long long*>(smem);
  const int q            = blockIdx.x;
  const int total        = nsrc * KO;
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    unsigned long long k = kNoKey;
    if (i < total) {
      const int h       = i / KO;
      const int64_t at  = h * src_stride + static_cast<int64_t>(q) * KO + i % KO;
      const long long v = src_i[at];
      if (v >= 0)
        k = (static_cast<unsigned long long>(static_cast<unsigned>(v)) << 32) | __float_as_uint(src_d[at]);
    }
    mk[i] = k;
  }
  __syncthreads();
  bitonic_sort(mk, P);  // by (id, distance): the first key of an id run is its nearest copy
  const int per = (P + kRoundThreads - 1) / kRoundThreads;
  const int i0  = threadIdx.x * per;
  unsigned long long mine[4096 / kRoundThreads];
  int cnt = 0;
  for (int i = i0; i < min(P, i0 + per); i++) {
    const unsigned long long k = mk[i];
    unsigned long long out     = kNoKey;
    if (k != kNoKey && (i == 0 || (mk[i - 1] >> 32) != (k >> 32)))
      out = ((k & 0xffffffffULL) << 32) | (k >> 32);
    mine[cnt++] = out;
  }
  __syncthreads();
  cnt = 0;
  for (int i = i0; i < min(P, i0 + per); i++)
    mk[i] = mine[cnt++];
  __syncthreads();
  bitonic_sort(mk, P);  // by (distance, id)
  long long* pb = si + static_cast<int64_t>(q) * KO;
  float* pd     = sd + static_cast<int64_t>(q) * KO;
  for (int i = threadIdx.x; i < KO; i += blockDim.x) {
    const unsigned long long k = mk[i];
    pb[i] = k == kNoKey ? -1 : static_cast<long long>(static_cast<unsigned>(k & 0xffffffffULL));
    pd[i] = k == kNoKey ? INFINITY : __uint_as_float(static_cast<unsigned>(k >> 32));
  }
}

}  // namespace

size_t round_smem_bytes(const round_args& a) { return sizeof(int) * round_layout(a).words; }

namespace {
template <bool kRows, bool kDealt, int kThreads>
void launch_round(const round_args& a, cudaStream_t s)
{
  round_kernel<kRows, kDealt, kThreads><<<a.m, kThreads, round_smem_bytes(a), s>>>(a);
}
template <bool kRows, bool kDealt>
void launch_round(const round_args& a, cudaStream_t s)
{
  if (a.threads >= 512)
    launch_round<kRows, kDealt, 512>(a, s);
  else if (a.threads >= 256)
    launch_round<kRows, kDealt, 256>(a, s);
  else
    launch_round<kRows, kDealt, 128>(a, s);
}
template <bool kRows, bool kDealt>
void allow_smem(int b)
{
  cudaFuncSetAttribute(round_kernel<kRows, kDealt, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, b);
  cudaFuncSetAttribute(round_kernel<kRows, kDealt, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, b);
  cudaFuncSetAttribute(round_kernel<kRows, kDealt, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, b);
}
bool dealt(const round_args& a)
{
  return a.table_map.ptrs != nullptr || a.sketch_map.ptrs != nullptr || a.vector_map.ptrs != nullptr;
}
}  // namespace

void round_allow_smem(size_t bytes)
{
  const int b = static_cast<int>(bytes);
  allow_smem<false, false>(b);
  allow_smem<true, false>(b);
  allow_smem<false, true>(b);
  allow_smem<true, true>(b);
}

void round_lists(const round_args& a, cudaStream_t s)
{
  if (a.m <= 0) return;
  if (dealt(a))
    launch_round<false, true>(a, s);
  else
    launch_round<false, false>(a, s);
}

void round_rows(const round_args& a, cudaStream_t s)
{
  if (a.m <= 0) return;
  if (dealt(a))
    launch_round<true, true>(a, s);
  else
    launch_round<true, false>(a, s);
}

void final_rerank(const long long* si, int KO, int R, const __half* vectors, row_map vector_map, int D,
                  const float* Q, int k, int m, long long* bi, float* bd, long long* stats,
                  cudaStream_t s)
{
  if (m <= 0) return;
  int P = 2;
  while (P < k)
    P <<= 1;
  const size_t words = 2 * static_cast<size_t>((k + R + 1) & ~1) + 2 * static_cast<size_t>(std::max(2 * P, 64)) +
                       2 * static_cast<size_t>((R + 3) & ~3) + ((D + 63) & ~63) + 256 + 16 + 8;
  final_rerank_kernel<<<m, kRoundThreads, sizeof(int) * words, s>>>(si, KO, R, vectors, vector_map, D, Q,
                                                                    k, P, bi, bd, stats);
}

void merge_kept(const long long* src_i, const float* src_d, int nsrc, int64_t src_stride, int KO,
                int P, int m, long long* si, float* sd, cudaStream_t s)
{
  if (m <= 0) return;
  const size_t smem = sizeof(int) * (2 * static_cast<size_t>(P) + 16);
  if (smem > (48 << 10))  // per device and context, so asked for whenever it is needed
    cudaFuncSetAttribute(merge_kept_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 4096 + 64);
  merge_kept_kernel<<<m, kRoundThreads, smem, s>>>(src_i, src_d, nsrc, src_stride, KO, P, si, sd);
}

}  // namespace octex_b200::kernels
