// Preparation kernels of a batch (sm_100a): padding, centring, projection, cell codes, cell lookup, best k.
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
// (search.cu:321-341): a block takes kCenterRows queries, their centred copies sit in shared
// memory, a thread owns one sketch coordinate of eight of them, so an element of the basis is read
// once per eight queries; each (query, coordinate) sum runs over the dimensions in order.
constexpr int kCenterRows = 16;
__global__ void __launch_bounds__(128) center_sketch_kernel(const float* __restrict__ q,
                                                            const float* __restrict__ mean,
                                                            const float* __restrict__ basis,
                                                            int m,
                                                            int D,
                                                            int S,
                                                            __half* __restrict__ qh,
                                                            int ldq,
                                                            float* __restrict__ qs)
{
  extern __shared__ __align__(16) float qc[];  // [D][kCenterRows]: the rows of a dimension side by side
  const int row0 = blockIdx.x * kCenterRows;
  const int rows = min(kCenterRows, m - row0);
  // fp16 copies, consecutive threads on consecutive dimensions
  for (int i = threadIdx.x; i < rows * ldq; i += blockDim.x) {
    const int r = i / ldq, d = i - r * ldq;
    const float v = d < D ? __fsub_rn(q[static_cast<int64_t>(row0 + r) * D + d], mean[d]) : 0.f;
    qh[static_cast<int64_t>(row0 + r) * ldq + d] = __float2half_rn(v);
  }
  // fp32 copies for the sketch, stored in the order the threads run (row fastest)
  for (int i = threadIdx.x; i < kCenterRows * D; i += blockDim.x) {
    const int r = i % kCenterRows, d = i / kCenterRows;
    qc[d * kCenterRows + r] = r < rows ? __fsub_rn(q[static_cast<int64_t>(row0 + r) * D + d], mean[d]) : 0.f;
  }
  __syncthreads();
  // an item = (group of 8 rows, sketch coordinate): 8 sums, each over the dimensions in order
  constexpr int kGroups = kCenterRows / 8;
  for (int item = threadIdx.x; item < kGroups * S; item += blockDim.x) {
    const int g = item / S, s = item - g * S;
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; r++)
      acc[r] = 0.f;
    const float* col = basis + s;
    const float* own = qc + 8 * g;
    int d = 0;
    for (; d + 8 <= D; d += 8) {
      float b[8];
#pragma unroll
      for (int u = 0; u < 8; u++)
        b[u] = __ldg(col + static_cast<int64_t>(d + u) * S);
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const float4 x0 = *reinterpret_cast<const float4*>(own + (d + u) * kCenterRows);
        const float4 x1 = *reinterpret_cast<const float4*>(own + (d + u) * kCenterRows + 4);
        acc[0] = __fmaf_rn(x0.x, b[u], acc[0]);
        acc[1] = __fmaf_rn(x0.y, b[u], acc[1]);
        acc[2] = __fmaf_rn(x0.z, b[u], acc[2]);
        acc[3] = __fmaf_rn(x0.w, b[u], acc[3]);
        acc[4] = __fmaf_rn(x1.x, b[u], acc[4]);
        acc[5] = __fmaf_rn(x1.y, b[u], acc[5]);
        acc[6] = __fmaf_rn(x1.z, b[u], acc[6]);
        acc[7] = __fmaf_rn(x1.w, b[u], acc[7]);
      }
    }
    for (; d < D; d++) {
      const float b = __ldg(col + static_cast<int64_t>(d) * S);
#pragma unroll
      for (int r = 0; r < 8; r++)
        acc[r] = __fmaf_rn(own[d * kCenterRows + r], b, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 8; r++)
      if (8 * g + r < rows) qs[static_cast<int64_t>(row0 + 8 * g + r) * S + s] = acc[r];
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
  // rows small against the spacing take the short decode, as in the projection's epilogue
  const float tame_y = inv_f > 0.f ? 0.99f * kTameLimit / inv_f : 0.f;
  bool wild          = false;
#pragma unroll
  for (int i = 0; i < 8 * B; i++) {
    v[i] = y[t * 8 * B + i];
    wild = wild || !(fabsf(v[i]) < tame_y);
  }
  codes[t] = wild ? cell_code<B>(v, inv_f) : cell_code_tame<B>(v, inv_f);
}

// ---- cell lookup -----------------------------------------------------------------------------

// The cells of a (copy, level) in an open-addressing table (slot = low bits of the 64-bit code,
// linear probing): what the reference keeps as a bucket-bound array plus a key array
// (search_kernels.cuh:100-126), re-laid so that a lookup costs one random 32-byte sector instead of
// two dependent ones. Built once when the index is placed.
__global__ void fill_cell_tables_kernel(const long long* __restrict__ keys,
                                        int64_t mmax,
                                        const int* __restrict__ ncells,
                                        const long long* __restrict__ toff,
                                        const int* __restrict__ tmask,
                                        cell_slot* __restrict__ table)
{
  const int cl = blockIdx.y;
  const int p  = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= ncells[cl]) return;
  const long long key = keys[static_cast<int64_t>(cl) * mmax + p];
  const unsigned mask = static_cast<unsigned>(tmask[cl]);
  cell_slot* mine     = table + toff[cl];
  unsigned s          = static_cast<unsigned>(key) & mask;
  for (unsigned probe = 0; probe <= mask; probe++) {
    if (atomicCAS(&mine[s].row, -1, p) == -1) {
      mine[s].key = key;  // nobody reads the table before this kernel is over
      return;
    }
    s = (s + 1) & mask;
  }
}

// search_kernels.cuh:100-126: the finest level whose cell holds a list. One thread per
// (query, copy). The codes of all levels are already there, so the home slot of every level is
// fetched at once (one 16-byte load each): one memory round trip for the common case instead of
// two per level tried. The answer is that of the level-by-level walk.
constexpr int kProbeLevels = 8;  // levels handled in one sweep; more are walked in further sweeps
__global__ void probe_kernel(const long long* __restrict__ codes,
                             int64_t pairs,
                             int C,
                             int L,
                             const cell_slot* __restrict__ table,
                             const long long* __restrict__ toff,
                             const int* __restrict__ tmask,
                             const int* __restrict__ base,
                             const unsigned char* __restrict__ level_on,
                             int list_len,
                             int lr,
                             int2* __restrict__ seg,
                             long long* __restrict__ stats)
{
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= pairs) return;
  const int c = static_cast<int>(t % C);
  int2 sg     = make_int2(0, 0);
  long long tried = 0, scanned = 0;
  bool found = false;
  for (int j0 = 0; j0 < L && !found; j0 += kProbeLevels) {
    long long h[kProbeLevels];
    int4 first[kProbeLevels];  // the home slot: (key low, key high, row, pad)
    bool on[kProbeLevels];
#pragma unroll
    for (int u = 0; u < kProbeLevels; u++) {
      const int j = j0 + u;
      on[u]       = j < L && (level_on == nullptr || level_on[c * L + j]);
      h[u]        = 0;
      first[u]    = make_int4(0, 0, -1, 0);
      if (on[u]) {
        const int cl = c * L + j;
        h[u]         = codes[t * L + j];
        first[u]     = __ldg(reinterpret_cast<const int4*>(table + toff[cl] +
                                                       (static_cast<unsigned>(h[u]) & static_cast<unsigned>(tmask[cl]))));
      }
    }
#pragma unroll
    for (int u = 0; u < kProbeLevels; u++) {
      if (found || !on[u]) continue;
      tried++;
      const int cl        = c * L + j0 + u;
      const unsigned mask = static_cast<unsigned>(tmask[cl]);
      const cell_slot* tb = table + toff[cl];
      unsigned s          = static_cast<unsigned>(h[u]) & mask;
      int4 e              = first[u];
      for (unsigned probe = 0; probe <= mask; probe++) {
        scanned++;
        if (e.z < 0) break;  // an empty slot ends the run: the cell does not exist
        const long long key = (static_cast<long long>(e.y) << 32) | static_cast<unsigned>(e.x);
        if (key == h[u]) {
          sg    = make_int2((base[cl] + e.z) * list_len, lr);
          found = true;
          break;
        }
        s = (s + 1) & mask;
        e = __ldg(reinterpret_cast<const int4*>(tb + s));
      }
    }
  }
  seg[t] = sg;
  if (stats != nullptr) {
    const int64_t q = t / C;
    atomicAdd(reinterpret_cast<unsigned long long*>(stats + q * 8), static_cast<unsigned long long>(tried));
    atomicAdd(reinterpret_cast<unsigned long long*>(stats + q * 8 + 1), static_cast<unsigned long long>(scanned));
  }
}

// The part of the sketch distance that depends on the row alone. The reference scores
// sum_k (c_k s_k - q_k)^2 in fp32 per candidate (search_kernels.cuh:228-251); expanded,
// sum_k (c_k s_k)^2 is a constant of the row and is computed here once, when the index is placed.
__global__ void sketch_row_norms_kernel(const signed char* __restrict__ codes,
                                        const float* __restrict__ scale,
                                        int64_t rows,
                                        int S,
                                        float* __restrict__ norm)
{
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(codes + r * S);
  float acc        = 0.f;
  for (int c = 0; c < S / 16; c++) {
    const uint4 v        = src[c];
    const unsigned wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int t = 0; t < 16; t++) {
      const int code = static_cast<signed char>((wd[t >> 2] >> (8 * (t & 3))) & 0xffu);
      const float x  = __fmul_rn(static_cast<float>(code), scale[c * 16 + t]);
      acc            = __fmaf_rn(x, x, acc);
    }
  }
  norm[r] = acc;
}

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
  const size_t smem = sizeof(float) * kCenterRows * D;
  // the opt-in belongs to the current device's context: asked for at every launch that needs it
  // (a host-side call, no stream work), so a process that places indexes on several GPUs is covered
  if (smem > (48 << 10))
    cudaFuncSetAttribute(center_sketch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  center_sketch_kernel<<<(m + kCenterRows - 1) / kCenterRows, 128, smem, s>>>(q, mean, basis, m, D, S, qh,
                                                                             ldq, qs);
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

void build_cell_tables(const long long* keys, int64_t mmax, const int* ncells, const long long* toff,
                       const int* tmask, int CL, cell_slot* table, cudaStream_t s)
{
  if (CL <= 0 || mmax <= 0) return;
  dim3 grid(blocks_for(mmax, 256), static_cast<unsigned>(CL));
  fill_cell_tables_kernel<<<grid, 256, 0, s>>>(keys, mmax, ncells, toff, tmask, table);
}

void probe(const long long* codes, int m, int C, int L, const cell_slot* table, const long long* toff,
           const int* tmask, const int* base, const unsigned char* level_on, int list_len, int lr,
           int2* seg, long long* stats, cudaStream_t s)
{
  const int64_t pairs = static_cast<int64_t>(m) * C;
  if (pairs <= 0) return;
  probe_kernel<<<blocks_for(pairs, 256), 256, 0, s>>>(codes, pairs, C, L, table, toff, tmask, base, level_on,
                                                      list_len, lr, seg, stats);
}

void sketch_row_norms(const signed char* codes, const float* scale, int64_t rows, int S, float* norm,
                      cudaStream_t s)
{
  if (rows <= 0) return;
  sketch_row_norms_kernel<<<blocks_for(rows, 128), 128, 0, s>>>(codes, scale, rows, S, norm);
}

void take_k(const long long* si, const float* sd, int KO, int k, int m, long long* bi, float* bd,
            cudaStream_t s)
{
  if (m <= 0) return;
  take_k_kernel<<<blocks_for(static_cast<int64_t>(m) * k, 256), 256, 0, s>>>(si, sd, KO, k, m, bi, bd);
}

}  // namespace octex_b200::kernels
