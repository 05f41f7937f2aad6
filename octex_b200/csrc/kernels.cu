// Search kernels (sm_100a). One thread block per query for every per-query step.
//
// Semantics follow the reference's kernels (hpdic/octex,
// cpp/src/neighbors/octex/detail/search_kernels.cuh); each kernel cites the lines it answers.
// The organisation is different: the cell codes of all levels are produced where the projected
// coordinates are produced, and each round (gather, dedup, sketch scoring, selection, exact
// rerank, merge into the kept list, and for waves the choice of start points) is one kernel that
// keeps a query's candidates in shared memory from the first list entry to the kept list.

#include "kernels.hpp"

#include "e8.cuh"

#include <cfloat>
#include <cmath>

namespace octex_b200::kernels {

namespace {

constexpr unsigned kIdHash = 2654435761u;
constexpr unsigned long long kNoKey = ~0ULL;

inline unsigned blocks_for(int64_t total, int threads)
{
  return static_cast<unsigned>((total + threads - 1) / threads);
}

// ---- padding, centring, sketch-space query -------------------------------------------------

// search_kernels.cuh:72-78
__global__ void pad_rows_kernel(float* __restrict__ q, int from, int m, int D)
{
  const int64_t t     = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(m - from) * D;
  if (t >= total) return;
  q[static_cast<int64_t>(from) * D + t] = q[t % D];
}

// Centre (search_kernels.cuh:57-69) fused with the sketch-space projection of the query
// (search.cu:321-341): one block per query, the centred query in shared memory, thread s owns
// sketch coordinate s.
__global__ void center_sketch_kernel(const float* __restrict__ q,
                                     const float* __restrict__ mean,
                                     const float* __restrict__ basis,
                                     int D,
                                     int S,
                                     __half* __restrict__ qh,
                                     int ldq,
                                     float* __restrict__ qs)
{
  extern __shared__ float qc[];
  const int row = blockIdx.x;
  for (int d = threadIdx.x; d < ldq; d += blockDim.x) {
    float v = 0.f;
    if (d < D) {
      v     = __fsub_rn(q[static_cast<int64_t>(row) * D + d], mean[d]);
      qc[d] = v;
    }
    qh[static_cast<int64_t>(row) * ldq + d] = __float2half_rn(v);
  }
  __syncthreads();
  for (int s = threadIdx.x; s < S; s += blockDim.x) {
    float acc = 0.f;
    for (int d = 0; d < D; d++)
      acc = __fmaf_rn(qc[d], basis[static_cast<int64_t>(d) * S + s], acc);
    qs[static_cast<int64_t>(row) * S + s] = acc;
  }
}

// ---- projection in the checker's summation order ---------------------------------------------

// Y = half(fp32(qh . ut^T) + shift), search.cu:303-320. 64 x 64 output tile per block, 16 x 16
// threads with 4 x 4 outputs each; every output accumulates its dot product with one fused
// multiply-add per dimension in dimension order, which is the order the CPU checker uses, so the
// result is comparable bit for bit. The tensor-core projection of the search path is checked
// against this one.
constexpr int kOrdTile = 64, kOrdK = 32;
__global__ void __launch_bounds__(256) project_ordered_kernel(const __half* __restrict__ qh,
                                                              int ldq,
                                                              const __half* __restrict__ ut,
                                                              int ldu,
                                                              const __half* __restrict__ shift,
                                                              int m,
                                                              int N,
                                                              int D,
                                                              __half* __restrict__ Y)
{
  __shared__ float sa[kOrdK][kOrdTile + 1];
  __shared__ float sb[kOrdK][kOrdTile + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * kOrdTile, col0 = blockIdx.x * kOrdTile;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < D; k0 += kOrdK) {
    for (int i = threadIdx.x; i < kOrdTile * kOrdK; i += 256) {
      const int r = i / kOrdK, k = i % kOrdK;
      float a = 0.f, b = 0.f;
      if (k0 + k < D) {
        if (row0 + r < m) a = __half2float(qh[static_cast<int64_t>(row0 + r) * ldq + k0 + k]);
        if (col0 + r < N) b = __half2float(ut[static_cast<int64_t>(col0 + r) * ldu + k0 + k]);
      }
      sa[k][r] = a;
      sb[k][r] = b;
    }
    __syncthreads();
    const int kk = min(kOrdK, D - k0);
    for (int k = 0; k < kk; k++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        a[i] = sa[k][ty * 4 + i];
        b[i] = sb[k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
          acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = row0 + ty * 4 + i;
    if (r >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int c = col0 + tx * 4 + j;
      if (c < N)
        Y[static_cast<int64_t>(r) * N + c] =
          __float2half_rn(__fadd_rn(acc[i][j], __half2float(shift[c])));
    }
  }
}

// ---- cell codes of all levels from projected coordinates -----------------------------------

template <int B>
__global__ void decode_codes_kernel(const __half* __restrict__ Y,
                                    int64_t pairs,
                                    int C,
                                    int L,
                                    const float* __restrict__ inv_f,
                                    const unsigned char* __restrict__ level_on,
                                    long long* __restrict__ codes)
{
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= pairs) return;
  const int c = static_cast<int>(t % C);
  float y[8 * B];
  const uint4* yp = reinterpret_cast<const uint4*>(Y + t * 8 * B);
#pragma unroll
  for (int i = 0; i < B; i++) {
    const uint4 v     = yp[i];
    const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 f   = __half22float2(h2[j]);
      y[8 * i + 2 * j] = f.x;
      y[8 * i + 2 * j + 1] = f.y;
    }
  }
  for (int j = 0; j < L; j++) {
    long long h = 0;
    if (level_on == nullptr || level_on[c * L + j]) h = cell_code<B>(y, inv_f[j]);
    codes[t * L + j] = h;
  }
}

// Cell code of rows of 8 * B float32 coordinates at one scale (the device function on its own,
// for checks against other implementations of the decode).
template <int B>
__global__ void cell_codes_f32_kernel(const float* __restrict__ y, int64_t n, float inv_f,
                                      long long* __restrict__ codes)
{
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= n) return;
  float v[8 * B];
#pragma unroll
  for (int i = 0; i < 8 * B; i++)
    v[i] = y[t * 8 * B + i];
  codes[t] = cell_code<B>(v, inv_f);
}

// ---- cell lookup -----------------------------------------------------------------------------

// search_kernels.cuh:100-126: the finest level whose cell holds a list. One thread per
// (query, copy); the codes of all levels are already there, so a level costs two dependent
// reads (bucket bounds, then the short key scan) and no arithmetic.
__global__ void probe_kernel(const long long* __restrict__ codes,
                             int64_t pairs,
                             int C,
                             int L,
                             const int* __restrict__ offsets,
                             int64_t T1,
                             const long long* __restrict__ keys,
                             int64_t mmax,
                             const int* __restrict__ base,
                             const unsigned char* __restrict__ level_on,
                             int list_len,
                             int lr,
                             int log_buckets,
                             int2* __restrict__ seg,
                             long long* __restrict__ stats)
{
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= pairs) return;
  const int c             = static_cast<int>(t % C);
  const long long bmask   = (1LL << log_buckets) - 1;
  int2 sg                 = make_int2(0, 0);
  long long tried = 0, scanned = 0;
  for (int j = 0; j < L; j++) {
    if (level_on != nullptr && !level_on[c * L + j]) continue;
    const long long h   = codes[t * L + j];
    const int64_t cl    = static_cast<int64_t>(c) * L + j;
    const int* o        = offsets + cl * T1 + static_cast<int>(h & bmask);
    const int lo = o[0], hi = o[1];
    const long long* kk = keys + cl * mmax;
    tried++;
    bool found = false;
    for (int p = lo; p < hi; p++) {
      scanned++;
      if (kk[p] == h) {
        sg    = make_int2((base[cl] + p) * list_len, lr);
        found = true;
        break;
      }
    }
    if (found) break;
  }
  seg[t] = sg;
  if (stats != nullptr) {
    const int64_t q = t / C;
    atomicAdd(reinterpret_cast<unsigned long long*>(stats + q * 8), static_cast<unsigned long long>(tried));
    atomicAdd(reinterpret_cast<unsigned long long*>(stats + q * 8 + 1), static_cast<unsigned long long>(scanned));
  }
}

}  // namespace

// ---- one round of a query --------------------------------------------------------------------

namespace {

/// Offsets (in 4-byte words) of the regions of a round block's shared memory.
struct round_layout {
  int table, cand, dist, key, sid, sdv, qv, sc, fq, st, pre, hist, wsum, ctrl, words;
  __host__ __device__ explicit round_layout(const round_args& a)
  {
    const int in_smem = a.cand_global == nullptr ? a.nmax : 0;
    const int rm      = a.sketch_rank ? a.KO : a.R;
    int at            = 0;
    auto take         = [&](int n) {
      int o = at;
      at += (n + 1) & ~1;  // keep every region 8-byte aligned
      return o;
    };
    table = take(a.ht_slots);
    cand  = take(in_smem);
    dist  = take(in_smem);
    key   = take(2 * a.P);
    sid   = take(rm);
    sdv   = take(rm);
    qv    = take(a.sw);
    sc    = take(a.sw);
    fq    = take(a.D);
    st    = take(a.nseg);
    pre   = take(a.nseg + 1);
    hist  = take(256);
    wsum  = take(16);
    ctrl  = take(8);
    words = at;
  }
};

__device__ __forceinline__ int hash_log_of(int total, int log_cap)
{
  // smallest e in [kMinLogHash, log_cap] with 2^e >= 1.5 * total (search_kernels.cuh:33-38)
  const int need = (3 * total + 1) / 2;
  int e          = kMinLogHash;
  while (e < log_cap && (1 << e) < need)
    e++;
  return e;
}

/// Exclusive prefix of v over the block (kRoundThreads threads); total = the sum.
__device__ __forceinline__ int block_scan(int v, int* wsum, int& total)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int nw = kRoundThreads / 32;
  int inc = v;
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
          const bool up                = (i & size) == 0;
          const unsigned long long a   = key[i], b = key[j];
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

/// The R smallest of n candidates by (distance bits, id): 8-bit radix passes over the 64-bit key
/// from the top, stopping at the first pass whose bucket is taken whole. Equal sketch distances
/// at the cut go to the smaller ids (search_kernels.cuh:259-322 takes them in any order).
/// Selected ids and distances land in sid / sdv in no particular order; ctrl[0] = their count.
__device__ __forceinline__ void select_smallest(const int* cand,
                                                const float* dist,
                                                int n,
                                                int R,
                                                int* sid,
                                                float* sdv,
                                                unsigned* hist,
                                                int* ctrl)
{
  if (n <= R) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      sid[i] = cand[i];
      sdv[i] = dist[i];
    }
    if (threadIdx.x == 0) ctrl[0] = n;
    __syncthreads();
    return;
  }
  unsigned long long prefix = 0, mask = 0;
  int need = R;
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x)
      hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const unsigned long long k = rank_key(dist[i], static_cast<unsigned>(cand[i]));
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1u);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // lane l owns digits 8l .. 8l+7: find the digit at which the running count reaches `need`
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
      const bool here = before < static_cast<unsigned>(need) && inc >= static_cast<unsigned>(need);
      if (here) {
        unsigned cum = before;
        int d        = 0;
#pragma unroll
        for (int t = 0; t < 8; t++) {
          if (cum + h[t] >= static_cast<unsigned>(need)) {
            d = t;
            break;
          }
          cum += h[t];
        }
        ctrl[1] = 8 * lane + d;                      // digit
        ctrl[2] = need - static_cast<int>(cum);      // still needed from that bucket
        ctrl[3] = static_cast<int>(h[d]);            // bucket size
      }
    }
    __syncthreads();
    const int digit = ctrl[1], left = ctrl[2], bucket = ctrl[3];
    prefix |= static_cast<unsigned long long>(digit) << shift;
    mask |= 255ULL << shift;
    need = left;
    __syncthreads();
    if (bucket == left) break;
  }
  if (threadIdx.x == 0) ctrl[0] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long k = rank_key(dist[i], static_cast<unsigned>(cand[i]));
    if ((k & mask) <= prefix) {
      const int s = atomicAdd(&ctrl[0], 1);
      if (s < R) {
        sid[s] = cand[i];
        sdv[s] = dist[i];
      }
    }
  }
  __syncthreads();
}

/// Squared distances of the fp16 rows sid[0, ns) to the fp32 query fq, written over sdv.
/// Summation order (shared with the CPU checker): element pair k feeds partial sum k mod 32 with
/// two fused multiply-adds; a butterfly over the 32 partial sums (search_kernels.cuh:325-342 is
/// the reference's warp-per-row form of the same sum). Eight lanes own a row here, each reading
/// 16 bytes per step, so that a warp keeps four rows and 512 bytes in flight.
__device__ __forceinline__ void exact_distances(
  const int* sid, int ns, const __half* __restrict__ vectors, int D, const float* fq, float* sdv)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((D & 7) == 0) {
    const int sub = lane & 7, grp = lane >> 3;
    for (int j0 = warp * 4; j0 < ns; j0 += nw * 4) {
      const int j = j0 + grp;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (j < ns) {
        const uint4* row = reinterpret_cast<const uint4*>(vectors + static_cast<int64_t>(sid[j]) * D);
        for (int h0 = 8 * sub; h0 < D; h0 += 64) {
          const uint4 v     = __ldg(row + (h0 >> 3));
          const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const float2 x = __half22float2(h2[t]);
            const float a  = __fsub_rn(x.x, fq[h0 + 2 * t]);
            const float b  = __fsub_rn(x.y, fq[h0 + 2 * t + 1]);
            acc[t]         = __fmaf_rn(b, b, __fmaf_rn(a, a, acc[t]));
          }
        }
      }
#pragma unroll
      for (int o = 4; o; o >>= 1)
#pragma unroll
        for (int t = 0; t < 4; t++)
          acc[t] = __fadd_rn(acc[t], __shfl_xor_sync(0xffffffffu, acc[t], o));
      if (j < ns && sub == 0)
        sdv[j] = __fadd_rn(__fadd_rn(acc[0], acc[2]), __fadd_rn(acc[1], acc[3]));
    }
  } else {
    for (int j = warp; j < ns; j += nw) {
      const __half2* row = reinterpret_cast<const __half2*>(vectors + static_cast<int64_t>(sid[j]) * D);
      float acc = 0.f;
      for (int k = lane; k < D / 2; k += 32) {
        const float2 x = __half22float2(row[k]);
        const float a  = __fsub_rn(x.x, fq[2 * k]);
        const float b  = __fsub_rn(x.y, fq[2 * k + 1]);
        acc            = __fmaf_rn(b, b, __fmaf_rn(a, a, acc));
      }
#pragma unroll
      for (int o = 16; o; o >>= 1)
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
      if (lane == 0) sdv[j] = acc;
    }
  }
  __syncthreads();
}

/// Merge ns new (distance, id) pairs into the kept list of KO: ascending distinct keys, padded
/// with (-1, +inf) (search_kernels.cuh:372-415; the copy-out is a block-wide compaction here).
__device__ __forceinline__ void merge_into_kept(unsigned long long* key,
                                                int P,
                                                long long* pb,
                                                float* pd,
                                                int KO,
                                                bool fresh,
                                                const int* sid,
                                                const float* sdv,
                                                int ns,
                                                int* wsum)
{
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    unsigned long long k = kNoKey;
    if (i < KO) {
      if (!fresh && pb[i] >= 0) k = rank_key(pd[i], static_cast<unsigned>(pb[i]));
    } else if (i - KO < ns) {
      k = rank_key(sdv[i - KO], static_cast<unsigned>(sid[i - KO]));
    }
    key[i] = k;
  }
  __syncthreads();
  bitonic_sort(key, P);
  const int per = (P + kRoundThreads - 1) / kRoundThreads;
  const int i0  = threadIdx.x * per;
  int mine      = 0;
  for (int i = i0; i < min(P, i0 + per); i++) {
    const unsigned long long k = key[i];
    if (k != kNoKey && (i == 0 || key[i - 1] != k)) mine++;
  }
  int total     = 0;
  int at        = block_scan(mine, wsum, total);
  for (int i = i0; i < min(P, i0 + per); i++) {
    const unsigned long long k = key[i];
    if (k != kNoKey && (i == 0 || key[i - 1] != k)) {
      if (at < KO) {
        pb[at] = static_cast<long long>(static_cast<unsigned>(k & 0xffffffffULL));
        pd[at] = __uint_as_float(static_cast<unsigned>(k >> 32));
      }
      at++;
    }
  }
  for (int o = total + threadIdx.x; o < KO; o += blockDim.x) {
    pb[o] = -1;
    pd[o] = INFINITY;
  }
}

template <bool kRows>
__global__ void __launch_bounds__(kRoundThreads) round_kernel(const round_args a)
{
  extern __shared__ __align__(16) int smem[];
  const round_layout lay(a);
  const int q = blockIdx.x;
  int* table              = smem + lay.table;
  int* cand               = a.cand_global ? a.cand_global + static_cast<int64_t>(q) * a.nmax : smem + lay.cand;
  float* dist             = a.dist_global ? a.dist_global + static_cast<int64_t>(q) * a.nmax
                                          : reinterpret_cast<float*>(smem + lay.dist);
  unsigned long long* key = reinterpret_cast<unsigned long long*>(smem + lay.key);
  int* sid                = smem + lay.sid;
  float* sdv              = reinterpret_cast<float*>(smem + lay.sdv);
  float* qv               = reinterpret_cast<float*>(smem + lay.qv);
  float* sc               = reinterpret_cast<float*>(smem + lay.sc);
  float* fq               = reinterpret_cast<float*>(smem + lay.fq);
  int* st                 = smem + lay.st;
  int* pre                = smem + lay.pre;
  unsigned* hist          = reinterpret_cast<unsigned*>(smem + lay.hist);
  int* wsum               = smem + lay.wsum;
  int* ctrl               = smem + lay.ctrl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int S = a.sw;
  long long* pb = a.si + static_cast<int64_t>(q) * a.KO;
  float* pd     = a.sd + static_cast<int64_t>(q) * a.KO;

  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    qv[i] = a.qs[static_cast<int64_t>(q) * S + i];
    sc[i] = a.scale[i];
  }
  if (!a.sketch_rank)
    for (int i = threadIdx.x; i < a.D; i += blockDim.x)
      fq[i] = a.Q[static_cast<int64_t>(q) * a.D + i];
  if (threadIdx.x == 0) ctrl[4] = 0;  // distinct ids

  int total = 0;
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
    const int per = (a.KO + kRoundThreads - 1) / kRoundThreads;
    const int i0  = threadIdx.x * per;
    unsigned fresh_bits = 0;
    int mine = 0;
    for (int i = i0; i < min(a.KO, i0 + per); i++) {
      const long long v = pb[i];
      bool f            = v >= 0;
      if (f) {
        unsigned h = (static_cast<unsigned>(v) * kIdHash) & (a.pick_slots - 1);
        for (int p = 0; p < a.pick_slots; p++) {
          const int t = table[h];
          if (t == -1) break;
          if (t == static_cast<int>(v)) {
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
    int at     = block_scan(mine, wsum, nfresh);
    for (int i = i0; i < min(a.KO, i0 + per); i++)
      if (fresh_bits & (1u << (i - i0))) {
        if (at < a.nseg) {
          const int v           = static_cast<int>(pb[i]);
          st[at]                = v;
          pdone[a.done_off + at] = v;
        }
        at++;
      }
    const int ns = min(nfresh, a.nseg);
    for (int o = ns + threadIdx.x; o < a.nseg; o += blockDim.x)
      pdone[a.done_off + o] = -1;
    total = ns * a.table_len;
    if (threadIdx.x == 0) ctrl[5] = ns;
    __syncthreads();
  } else {
    // exclusive prefix of the segment lengths (search_kernels.cuh:171-188)
    if (warp == 0) {
      int carry = 0;
      for (int c0 = 0; c0 < a.nseg; c0 += 32) {
        const int c   = c0 + lane;
        const int2 sl = c < a.nseg ? a.seg[static_cast<int64_t>(q) * a.nseg + c] : make_int2(0, 0);
        int v         = sl.y;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, v, o);
          if (lane >= o) v += u;
        }
        if (c < a.nseg) {
          pre[c] = carry + v - sl.y;
          st[c]  = sl.x;
        }
        carry += __shfl_sync(0xffffffffu, v, 31);
      }
      if (lane == 0) pre[a.nseg] = carry;
    }
    __syncthreads();
    total = pre[a.nseg];
  }

  // distinct ids through an open-addressing hash set (search_kernels.cuh:191-225)
  const int HT = 1 << hash_log_of(total, a.log_cap);
  for (int i = threadIdx.x; i < HT; i += blockDim.x)
    table[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    int v;
    if constexpr (kRows) {
      const int j = i / a.table_len;
      v = __ldg(a.table + static_cast<int64_t>(st[j]) * a.table_len + (i - j * a.table_len));
    } else {
      int lo = 0, hi = a.nseg - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (pre[mid] <= i)
          lo = mid;
        else
          hi = mid - 1;
      }
      v = __ldg(a.lists + static_cast<int64_t>(lo) * a.stride + st[lo] + (i - pre[lo]));
    }
    if (v < 0) continue;  // padding of a table row
    unsigned s = (static_cast<unsigned>(v) * kIdHash) & (HT - 1);
    for (int p = 0; p < HT; p++) {
      const int prev = atomicCAS(&table[s], -1, v);
      if (prev == -1) {
        const int slot = atomicAdd(&ctrl[4], 1);
        if (slot < a.nmax) cand[slot] = v;
        break;
      }
      if (prev == v) break;
      s = (s + 1) & (HT - 1);
    }
  }
  __syncthreads();
  const int n = min(ctrl[4], a.nmax);

  // int8 sketch distances (search_kernels.cuh:228-251): Lr lanes per row, one 16-byte chunk each
  int Lr = 1;
  while (Lr < S / 16 && Lr < 32)
    Lr <<= 1;
  const int G = 32 / Lr, sub = lane % Lr;
  for (int j0 = warp * G; j0 < n; j0 += nw * G) {
    const int j = j0 + lane / Lr;
    float d     = 0.f;
    if (j < n && sub * 16 < S) {
      const signed char* x = a.sketch + static_cast<int64_t>(cand[j]) * S + sub * 16;
      const int4 w         = __ldg(reinterpret_cast<const int4*>(x));
      const signed char* b = reinterpret_cast<const signed char*>(&w);
#pragma unroll
      for (int t = 0; t < 16; t++) {
        const int k   = sub * 16 + t;
        const float u = __fmaf_rn(static_cast<float>(b[t]), sc[k], -qv[k]);
        d             = __fmaf_rn(u, u, d);
      }
    }
    for (int o = Lr >> 1; o; o >>= 1)
      d = __fadd_rn(d, __shfl_xor_sync(0xffffffffu, d, o));
    if (j < n && sub == 0) dist[j] = d;
  }
  __syncthreads();
  if (a.tap_cand != nullptr) {
    for (int i = threadIdx.x; i < min(n, a.tap_cap); i += blockDim.x) {
      a.tap_cand[static_cast<int64_t>(q) * a.tap_cap + i] = cand[i];
      a.tap_dist[static_cast<int64_t>(q) * a.tap_cap + i] = dist[i];
    }
    if (threadIdx.x == 0) a.tap_n[q] = n;
  }

  // the nearest by sketch: reranked exactly, or kept as they are
  select_smallest(cand, dist, n, a.sketch_rank ? a.KO : a.R, sid, sdv, hist, ctrl);
  const int ns = min(ctrl[0], a.sketch_rank ? a.KO : a.R);
  if (!a.sketch_rank) exact_distances(sid, ns, a.vectors, a.D, fq, sdv);
  merge_into_kept(key, a.P, pb, pd, a.KO, a.fresh != 0, sid, sdv, ns, wsum);
  if (a.stats != nullptr && threadIdx.x == 0) {
    long long* s = a.stats + static_cast<int64_t>(q) * 8;
    if constexpr (kRows) {
      s[4] += ctrl[5];
      s[5] += n;
    } else {
      s[2] += total;
      s[3] += n;
    }
    if (!a.sketch_rank) s[6] += ns;
  }
}

}  // namespace

// ---- best k, cross-GPU merge -----------------------------------------------------------------

namespace {

// search_kernels.cuh:672-685
__global__ void take_k_kernel(const long long* __restrict__ si,
                              const float* __restrict__ sd,
                              int KO,
                              int k,
                              int m,
                              long long* __restrict__ bi,
                              float* __restrict__ bd)
{
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<int64_t>(m) * k) return;
  const int64_t q = t / k, j = t % k;
  bi[t] = si[q * KO + j];
  bd[t] = sd[q * KO + j];
}

// search_kernels.cuh:634-669: exact distances of the first R kept entries, best k of them.
__global__ void __launch_bounds__(kRoundThreads) final_rerank_kernel(const long long* __restrict__ si,
                                                                     int KO,
                                                                     int R,
                                                                     const __half* __restrict__ vectors,
                                                                     int D,
                                                                     const float* __restrict__ Q,
                                                                     int k,
                                                                     int P,
                                                                     long long* __restrict__ bi,
                                                                     float* __restrict__ bd,
                                                                     long long* __restrict__ stats)
{
  extern __shared__ __align__(16) int smem[];
  unsigned long long* key = reinterpret_cast<unsigned long long*>(smem);  // [P]
  int* sid                = smem + 2 * P;                                 // [R]
  float* sdv              = reinterpret_cast<float*>(sid + R);            // [R]
  float* fq               = sdv + R;                                      // [D]
  int* wsum               = reinterpret_cast<int*>(fq + D);               // [16]
  const int q             = blockIdx.x;
  const long long* ps     = si + static_cast<int64_t>(q) * KO;
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    fq[i] = Q[static_cast<int64_t>(q) * D + i];
  // the kept list is packed (valid entries first), so the valid ones among the first R are a prefix
  int mine = 0;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const long long v = ps[i];
    sid[i]            = static_cast<int>(v);
    if (v >= 0) mine++;
  }
  int ns = 0;
  block_scan(mine, wsum, ns);
  exact_distances(sid, ns, vectors, D, fq, sdv);
  merge_into_kept(key, P, bi + static_cast<int64_t>(q) * k, bd + static_cast<int64_t>(q) * k, k, true,
                  sid, sdv, ns, wsum);
  if (stats != nullptr && threadIdx.x == 0) stats[static_cast<int64_t>(q) * 8 + 6] += ns;
}

}  // namespace

namespace {

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
      const int h        = i / KO;
      const int64_t at   = h * src_stride + static_cast<int64_t>(q) * KO + i % KO;
      const long long v  = src_i[at];
      if (v >= 0)
        k = (static_cast<unsigned long long>(static_cast<unsigned>(v)) << 32) | __float_as_uint(src_d[at]);
    }
    mk[i] = k;
  }
  __syncthreads();
  bitonic_sort(mk, P);  // by (id, distance): the first key of an id run is its nearest copy
  const int per = (P + kRoundThreads - 1) / kRoundThreads;
  const int i0  = threadIdx.x * per;
  unsigned long long mine[16];
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

// ---- launchers ---------------------------------------------------------------------------------

void pad_rows(float* q, int from, int m, int D, cudaStream_t s)
{
  if (from >= m) return;
  pad_rows_kernel<<<blocks_for(static_cast<int64_t>(m - from) * D, 256), 256, 0, s>>>(q, from, m, D);
}

void center_sketch(const float* q, const float* mean, const float* basis, int m, int D, int S,
                   __half* qh, int ldq, float* qs, cudaStream_t s)
{
  if (m <= 0) return;
  center_sketch_kernel<<<m, 128, sizeof(float) * D, s>>>(q, mean, basis, D, S, qh, ldq, qs);
}

void project_ordered(const __half* qh, int ldq, const __half* ut, int ldu, const __half* shift,
                     int m, int N, int D, __half* Y, cudaStream_t s)
{
  if (m <= 0 || N <= 0) return;
  dim3 grid((N + kOrdTile - 1) / kOrdTile, (m + kOrdTile - 1) / kOrdTile);
  project_ordered_kernel<<<grid, 256, 0, s>>>(qh, ldq, ut, ldu, shift, m, N, D, Y);
}

void decode_codes(const __half* Y, int64_t pairs, int C, int blocks, int L, const float* inv_f,
                  const unsigned char* level_on, long long* codes, cudaStream_t s)
{
  if (pairs <= 0) return;
  const unsigned g = blocks_for(pairs, 128);
  switch (blocks) {
    case 1: decode_codes_kernel<1><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    case 2: decode_codes_kernel<2><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    case 3: decode_codes_kernel<3><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    case 4: decode_codes_kernel<4><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    case 5: decode_codes_kernel<5><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    case 6: decode_codes_kernel<6><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    case 8: decode_codes_kernel<8><<<g, 128, 0, s>>>(Y, pairs, C, L, inv_f, level_on, codes); break;
    default: break;  // the loader rejects other block counts
  }
}

void cell_codes_f32(const float* y, int64_t n, int blocks, float inv_f, long long* codes,
                    cudaStream_t s)
{
  if (n <= 0) return;
  const unsigned g = blocks_for(n, 128);
  switch (blocks) {
    case 1: cell_codes_f32_kernel<1><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    case 2: cell_codes_f32_kernel<2><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    case 3: cell_codes_f32_kernel<3><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    case 4: cell_codes_f32_kernel<4><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    case 5: cell_codes_f32_kernel<5><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    case 6: cell_codes_f32_kernel<6><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    case 8: cell_codes_f32_kernel<8><<<g, 128, 0, s>>>(y, n, inv_f, codes); break;
    default: break;
  }
}

void probe(const long long* codes, int m, int C, int L, const int* offsets, int64_t T1,
           const long long* keys, int64_t mmax, const int* base, const unsigned char* level_on,
           int list_len, int lr, int log_buckets, int2* seg, long long* stats, cudaStream_t s)
{
  const int64_t pairs = static_cast<int64_t>(m) * C;
  if (pairs <= 0) return;
  probe_kernel<<<blocks_for(pairs, 256), 256, 0, s>>>(codes, pairs, C, L, offsets, T1, keys, mmax,
                                                      base, level_on, list_len, lr, log_buckets,
                                                      seg, stats);
}

size_t round_smem_bytes(const round_args& a) { return sizeof(int) * round_layout(a).words; }

void round_allow_smem(size_t bytes)
{
  cudaFuncSetAttribute(round_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(bytes));
  cudaFuncSetAttribute(round_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(bytes));
}

void round_lists(const round_args& a, cudaStream_t s)
{
  if (a.m <= 0) return;
  round_kernel<false><<<a.m, kRoundThreads, round_smem_bytes(a), s>>>(a);
}

void round_rows(const round_args& a, cudaStream_t s)
{
  if (a.m <= 0) return;
  round_kernel<true><<<a.m, kRoundThreads, round_smem_bytes(a), s>>>(a);
}

void take_k(const long long* si, const float* sd, int KO, int k, int m, long long* bi, float* bd,
            cudaStream_t s)
{
  if (m <= 0) return;
  take_k_kernel<<<blocks_for(static_cast<int64_t>(m) * k, 256), 256, 0, s>>>(si, sd, KO, k, m, bi, bd);
}

void final_rerank(const long long* si, int KO, int R, const __half* vectors, int D, const float* Q,
                  int k, int m, long long* bi, float* bd, long long* stats, cudaStream_t s)
{
  if (m <= 0) return;
  int P = 2;
  while (P < k + R)
    P <<= 1;
  const size_t smem = sizeof(int) * (2 * P + 2 * R + D + 16);
  final_rerank_kernel<<<m, kRoundThreads, smem, s>>>(si, KO, R, vectors, D, Q, k, P, bi, bd, stats);
}

void merge_kept(const long long* src_i, const float* src_d, int nsrc, int64_t src_stride, int KO,
                int P, int m, long long* si, float* sd, cudaStream_t s)
{
  if (m <= 0) return;
  static bool allowed = false;
  const size_t smem   = sizeof(int) * (2 * P + 16);
  if (!allowed) {
    cudaFuncSetAttribute(merge_kept_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 4096 + 64);
    allowed = true;
  }
  merge_kept_kernel<<<m, kRoundThreads, smem, s>>>(src_i, src_d, nsrc, src_stride, KO, P, si, sd);
}

}  // namespace octex_b200::kernels
