// Index builder on one GPU: dataset -> format-1 index directory.
//
// Answers cpp/src/neighbors/octex/build.cu and detail/build_*.cuh of hpdic/octex for the build
// mode that needs none of its external libraries: member lists (the reference's
// index_params::member_lists / `--fast` path, detail/build_cells.cuh:874-1002), an exact neighbor
// table with the reverse-edge merge (detail/build_table.cuh:60-74,171-251,529-554), the sample PCA
// and seeded projections (detail/build_setup.cuh:40-175) and the int8 sketch (:177-264). Every
// array it writes has the dtype, shape and meaning the loader of this library and of the reference
// reads (docs/design.md:27-48). The pipeline is laid out for one B200: the fp16 dataset stays on
// the GPU for the whole build, a copy's cells are made by two radix sorts of all rows per spacing
// (distance to the own cell centre, then cell code: the runs are the cells with their members
// nearest first), and the neighbor table is a brute-force scan in tiles whose dot products
// accumulate fp16 products in fp32.

#include "build.hpp"

#include "e8.cuh"
#include "npy.hpp"
#include "sym_eigen.hpp"

#include "index_impl.hpp"
#include "kernels.hpp"
#include "search_impl.hpp"

#include <cub/cub.cuh>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <random>
#include <sstream>

namespace octex_b200 {

namespace {

inline unsigned grid_for(int64_t total, int threads)
{
  return static_cast<unsigned>((total + threads - 1) / threads);
}

template <typename T>
auto to_host(const void* dev, size_t count) -> std::vector<T>
{
  std::vector<T> out(count);
  if (count != 0) OCTEX_CUDA_TRY(cudaMemcpy(out.data(), dev, count * sizeof(T), cudaMemcpyDeviceToHost));
  return out;
}

// ---- dataset to fp16 on the device ---------------------------------------------------------------

__global__ void f32_to_f16_kernel(const float* __restrict__ x, int64_t n, __half* __restrict__ y)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2half_rn(x[i]);
}

// ---- sample PCA (build_setup.cuh:40-103) --------------------------------------------------------

// sum[k] += x[i * step, k] over the sampled rows of this block (fp64)
__global__ void sample_sum_kernel(const __half* __restrict__ x, int64_t ns, int64_t step, int D,
                                  double* __restrict__ sum)
{
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= D) return;
  const int64_t per = (ns + gridDim.y - 1) / gridDim.y;
  const int64_t i0 = per * blockIdx.y, i1 = min(ns, i0 + per);
  double acc = 0.0;
  for (int64_t i = i0; i < i1; i++)
    acc += static_cast<double>(__half2float(x[i * step * D + k]));
  atomicAdd(&sum[k], acc);
}

// g[a, b] += sum over the sampled rows of this block of (x[a] - mean[a]) (x[b] - mean[b]), fp64;
// the centring subtracts the fp32 mean in fp32 first, as the reference does
constexpr int kScatterTile = 16, kScatterRows = 64;
__global__ void __launch_bounds__(kScatterTile* kScatterTile)
  scatter_kernel(const __half* __restrict__ x, int64_t ns, int64_t step, int D, const float* __restrict__ mean,
                 double* __restrict__ g)
{
  __shared__ double sa[kScatterRows][kScatterTile + 1], sb[kScatterRows][kScatterTile + 1];
  const int ta = threadIdx.x % kScatterTile, tb = threadIdx.x / kScatterTile;
  const int a0 = blockIdx.x * kScatterTile, b0 = blockIdx.y * kScatterTile;
  if (b0 > a0) return;  // the matrix is symmetric: the lower triangle is mirrored on the host
  const int64_t per = (ns + gridDim.z - 1) / gridDim.z;
  const int64_t i0 = per * blockIdx.z, i1 = min(ns, i0 + per);
  double acc = 0.0;
  for (int64_t r0 = i0; r0 < i1; r0 += kScatterRows) {
    for (int t = threadIdx.x; t < kScatterRows * kScatterTile; t += blockDim.x) {
      const int r = t / kScatterTile, c = t % kScatterTile;
      const int64_t i = r0 + r;
      double va = 0.0, vb = 0.0;
      if (i < i1) {
        if (a0 + c < D) va = static_cast<double>(__fsub_rn(__half2float(x[i * step * D + a0 + c]), mean[a0 + c]));
        if (b0 + c < D) vb = static_cast<double>(__fsub_rn(__half2float(x[i * step * D + b0 + c]), mean[b0 + c]));
      }
      sa[r][c] = va;
      sb[r][c] = vb;
    }
    __syncthreads();
#pragma unroll 8
    for (int r = 0; r < kScatterRows; r++)
      acc += sa[r][ta] * sb[r][tb];
    __syncthreads();
  }
  if (a0 + ta < D && b0 + tb < D) atomicAdd(&g[static_cast<int64_t>(a0 + ta) * D + b0 + tb], acc);
}

struct pca_result {
  std::vector<float> mean;     // [D]
  std::vector<float> vectors;  // [D, D] row major: column k is the k-th principal direction
  std::vector<double> values;  // [D] eigenvalues of the sample scatter matrix, descending
  int64_t samples = 0;
};

auto sample_pca(const __half* x, int64_t n, int D, cudaStream_t s) -> pca_result
{
  constexpr int64_t kSampleRows = 200000;
  const int64_t step = std::max<int64_t>(1, n / kSampleRows);
  const int64_t ns   = (n + step - 1) / step;
  pca_result out;
  out.samples = ns;
  int dev     = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&dev));
  dbuf sum(dev, sizeof(double) * D), mean(dev, sizeof(float) * D), g(dev, sizeof(double) * D * D);
  OCTEX_CUDA_TRY(cudaMemsetAsync(sum.ptr, 0, sum.size, s));
  OCTEX_CUDA_TRY(cudaMemsetAsync(g.ptr, 0, g.size, s));
  sample_sum_kernel<<<dim3(grid_for(D, 128), 64), 128, 0, s>>>(x, ns, step, D, sum.as<double>());
  auto hs = to_host<double>(sum.ptr, D);
  out.mean.resize(D);
  for (int k = 0; k < D; k++)
    out.mean[k] = static_cast<float>(hs[k] / static_cast<double>(ns));
  OCTEX_CUDA_TRY(cudaMemcpyAsync(mean.ptr, out.mean.data(), mean.size, cudaMemcpyHostToDevice, s));
  const unsigned tiles = grid_for(D, kScatterTile);
  scatter_kernel<<<dim3(tiles, tiles, 64), kScatterTile * kScatterTile, 0, s>>>(x, ns, step, D, mean.as<float>(),
                                                                               g.as<double>());
  OCTEX_CUDA_TRY(cudaPeekAtLastError());
  auto hg = to_host<double>(g.ptr, static_cast<size_t>(D) * D);
  for (int a = 0; a < D; a++)
    for (int b = a + 1; b < D; b++)
      hg[static_cast<size_t>(a) * D + b] = hg[static_cast<size_t>(b) * D + a];  // mirror the computed triangle
  std::vector<double> val, vec;
  symmetric_eigen(hg, D, val, vec);
  out.values.resize(D);
  out.vectors.resize(static_cast<size_t>(D) * D);
  for (int k = 0; k < D; k++) {
    const int src = D - 1 - k;
    out.values[k] = std::max(val[src], 0.0);
    for (int r = 0; r < D; r++)
      out.vectors[static_cast<size_t>(r) * D + k] = static_cast<float>(vec[static_cast<size_t>(r) * D + src]);
  }
  return out;
}

// ---- seeded projections (build_setup.cuh:113-175) ------------------------------------------------

inline auto splitmix64(uint64_t z) -> uint64_t
{
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

/// proj [C, D, w], shift [C, w]: copy c rotates the top-p principal subspace into w dimensions by
/// the orthonormalised columns of a Gaussian [p, w] matrix (modified Gram-Schmidt) and divides by
/// the mean projected standard deviation of the sample; its shift is uniform in [0, 2). The
/// generator of copy c is std::mt19937_64 seeded with splitmix64(seed * 0x100000001B3 + c), the
/// reference's, so the same seed gives the same rotations where the standard library agrees.
void make_projections(pca_result const& pca, int D, int p, int w, int copies, uint64_t seed,
                      std::vector<float>& proj, std::vector<float>& shift)
{
  OCTEX_EXPECTS(p >= w, "octex: pca_dims must be at least 8 * blocks");
  OCTEX_EXPECTS(p <= D, "octex: pca_dims exceeds the dimension");
  proj.assign(static_cast<size_t>(copies) * D * w, 0.f);
  shift.assign(static_cast<size_t>(copies) * w, 0.f);
  std::vector<double> q(static_cast<size_t>(p) * w);
  const double denom = static_cast<double>(std::max<int64_t>(pca.samples - 1, 1));
  for (int c = 0; c < copies; c++) {
    std::mt19937_64 gen(splitmix64(seed * 0x100000001B3ULL + static_cast<uint64_t>(c)));
    std::normal_distribution<double> normal(0.0, 1.0);
    std::uniform_real_distribution<double> uniform(0.0, 2.0);
    for (auto& v : q)
      v = normal(gen);
    auto col_dot = [&](int a, int b) {
      double acc = 0.0;
      for (int r = 0; r < p; r++)
        acc += q[static_cast<size_t>(r) * w + a] * q[static_cast<size_t>(r) * w + b];
      return acc;
    };
    for (int s = 0; s < w; s++) {
      for (int t = 0; t < s; t++) {
        const double along = col_dot(s, t);
        for (int r = 0; r < p; r++)
          q[static_cast<size_t>(r) * w + s] -= along * q[static_cast<size_t>(r) * w + t];
      }
      const double length = std::sqrt(col_dot(s, s));
      for (int r = 0; r < p; r++)
        q[static_cast<size_t>(r) * w + s] /= length;
    }
    double sd = 0.0;
    for (int s = 0; s < w; s++) {
      double var = 0.0;
      for (int r = 0; r < p; r++)
        var += pca.values[r] * q[static_cast<size_t>(r) * w + s] * q[static_cast<size_t>(r) * w + s];
      sd += std::sqrt(var / denom);
    }
    sd /= w;
    float* u = proj.data() + static_cast<size_t>(c) * D * w;
    for (int k = 0; k < D; k++)
      for (int s = 0; s < w; s++) {
        double acc = 0.0;
        for (int r = 0; r < p; r++)
          acc += static_cast<double>(pca.vectors[static_cast<size_t>(k) * D + r]) * q[static_cast<size_t>(r) * w + s];
        u[static_cast<size_t>(k) * w + s] = static_cast<float>(acc / sd);
      }
    for (int s = 0; s < w; s++)
      shift[static_cast<size_t>(c) * w + s] = static_cast<float>(uniform(gen));
  }
}

// ---- y = (x - mean) @ m + bias for narrow m -------------------------------------------------------

// Rows of the fp16 dataset, centred in fp32, times a matrix of few columns (a copy's projection,
// the sketch basis): a block takes 64 rows and 32 columns, a thread 8 rows of one column; every
// sum runs over the dimensions in order with one fused multiply-add each.
constexpr int kRowsTile = 64, kColsTile = 32, kDimTile = 32;
__global__ void __launch_bounds__(256) rows_times_kernel(const __half* __restrict__ x,
                                                         const float* __restrict__ mean,
                                                         const float* __restrict__ m,  // [D, N]
                                                         const float* __restrict__ bias,  // [N] or null
                                                         int64_t n, int D, int N, float* __restrict__ y)
{
  __shared__ float xs[kDimTile][kRowsTile + 1];
  __shared__ float ms[kDimTile][kColsTile + 1];
  const int col = threadIdx.x % kColsTile, rg = threadIdx.x / kColsTile;  // 8 row groups of 8 rows
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsTile;
  const int col0     = blockIdx.y * kColsTile;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int d0 = 0; d0 < D; d0 += kDimTile) {
    for (int t = threadIdx.x; t < kRowsTile * kDimTile; t += 256) {
      const int r = t / kDimTile, d = t % kDimTile;
      float v = 0.f;
      if (row0 + r < n && d0 + d < D) v = __fsub_rn(__half2float(x[(row0 + r) * D + d0 + d]), mean[d0 + d]);
      xs[d][r] = v;
    }
    for (int t = threadIdx.x; t < kDimTile * kColsTile; t += 256) {
      const int d = t / kColsTile, c = t % kColsTile;
      ms[d][c] = (d0 + d < D && col0 + c < N) ? m[static_cast<int64_t>(d0 + d) * N + col0 + c] : 0.f;
    }
    __syncthreads();
    const int dd = min(kDimTile, D - d0);
    for (int d = 0; d < dd; d++) {
      const float b = ms[d][col];
#pragma unroll
      for (int r = 0; r < 8; r++)
        acc[r] = __fmaf_rn(xs[d][rg * 8 + r], b, acc[r]);
    }
    __syncthreads();
  }
  if (col0 + col >= N) return;
  const float add = bias != nullptr ? bias[col0 + col] : 0.f;
#pragma unroll
  for (int r = 0; r < 8; r++) {
    const int64_t row = row0 + rg * 8 + r;
    if (row < n) y[row * N + col0 + col] = __fadd_rn(acc[r], add);
  }
}

void rows_times(const __half* x, const float* mean, const float* m, const float* bias, int64_t n, int D,
                int N, float* y, cudaStream_t s)
{
  if (n <= 0) return;
  dim3 grid(grid_for(n, kRowsTile), grid_for(N, kColsTile));
  rows_times_kernel<<<grid, 256, 0, s>>>(x, mean, m, bias, n, D, N, y);
}

// ---- cells of one copy (build_cells.cuh:874-1002) -------------------------------------------------

// Per row: the code of its cell at one spacing and its squared distance to that cell's centre
// (the lattice point its coordinates round to, times the spacing).
template <int B>
__global__ void cell_of_rows_kernel(const float* __restrict__ y, int64_t n, float f, float inv_f,
                                    long long* __restrict__ code, float* __restrict__ dist)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v[8 * B];
#pragma unroll
  for (int k = 0; k < 8 * B; k++)
    v[k] = y[i * 8 * B + k];
  code[i] = cell_code<B>(v, inv_f);
  float d = 0.f;
#pragma unroll
  for (int j = 0; j < B; j++) {
    float xs[8], p[8];
#pragma unroll
    for (int k = 0; k < 8; k++)
      xs[k] = __fmul_rn(v[8 * j + k], inv_f);
    nearest_e8(xs, p);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const float e = __fsub_rn(v[8 * j + k], __fmul_rn(f, p[k]));
      d             = __fmaf_rn(e, e, d);
    }
  }
  dist[i] = d;
}

__global__ void iota_kernel(int32_t* v, int64_t n)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) v[i] = static_cast<int32_t>(i);
}

template <typename T>
__global__ void gather_kernel(const T* __restrict__ src, const int32_t* __restrict__ at, int64_t n,
                              T* __restrict__ dst)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[at[i]];
}

// keep[r] = the cell of run r stays (all cells of the coarsest spacing, else those of at least
// min_cell rows)
__global__ void keep_kernel(const int32_t* __restrict__ pop, int64_t runs, int min_cell, int32_t* __restrict__ keep)
{
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r < runs) keep[r] = pop[r] >= min_cell ? 1 : 0;
}

__global__ void compact_cells_kernel(const long long* __restrict__ ukey, const int32_t* __restrict__ start,
                                     const int32_t* __restrict__ pop, const int32_t* __restrict__ keep,
                                     const int32_t* __restrict__ slot, int64_t runs, long long* __restrict__ key,
                                     int32_t* __restrict__ kstart, int32_t* __restrict__ kpop)
{
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= runs || !keep[r]) return;
  key[slot[r]]    = ukey[r];
  kstart[slot[r]] = start[r];
  kpop[slot[r]]   = pop[r];
}

// lists[c, t] = row t of cell c in distance order, or its nearest row when the cell holds fewer
// (build_cells.cuh:784-793), written at the cell's place in (bucket, code) order
__global__ void cell_lists_kernel(const int32_t* __restrict__ sorted_rows, const int32_t* __restrict__ kstart,
                                  const int32_t* __restrict__ kpop, const int32_t* __restrict__ perm, int64_t cells,
                                  int l, int32_t* __restrict__ lists)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= cells * l) return;
  const int64_t at = i / l;
  const int t      = static_cast<int>(i % l);
  const int c      = perm[at];
  lists[i]         = sorted_rows[kstart[c] + (t < kpop[c] ? t : 0)];
}

__global__ void bucket_kernel(const long long* __restrict__ key, int64_t cells, long long mask, int32_t* __restrict__ bucket)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < cells) bucket[i] = static_cast<int32_t>(key[i] & mask);
}

// offsets[t] = first cell (in bucket order) whose bucket is >= t, t = 0 .. T
__global__ void bucket_bounds_kernel(const int32_t* __restrict__ sorted_bucket, int64_t cells, int64_t T1,
                                     int32_t* __restrict__ offsets)
{
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= T1) return;
  int64_t lo = 0, hi = cells;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (sorted_bucket[mid] < t)
      lo = mid + 1;
    else
      hi = mid;
  }
  offsets[t] = static_cast<int32_t>(lo);
}

/// What a copy contributes to the index arrays (host memory).
struct copy_cells {
  std::vector<int32_t> lists;    // rows of list_len ids, levels back to back
  std::vector<int64_t> keys;     // per level, cells[j] codes in (bucket, code) order, back to back
  std::vector<int32_t> offsets;  // per level T + 1 bucket bounds
  std::vector<int32_t> base;     // first list row of each level
  std::vector<int64_t> cells;    // cells of each level
};

/// Device scratch of the per-copy work, sized once for n rows.
struct cell_scratch {
  int64_t n = 0;
  dbuf y, code, code_alt, dist, dist_alt, rows, rows_alt, ukey, pop, start, keep, slot, key, kstart, kpop, bucket,
    bucket_alt, perm, perm_alt, runs, tmp, lists, offsets, skeys;
  size_t tmp_bytes = 0;
  cell_scratch(int dev, int64_t n_, int w, int l, int64_t T1) : n(n_)
  {
    y        = dbuf(dev, sizeof(float) * n * w);
    code     = dbuf(dev, sizeof(long long) * n);
    code_alt = dbuf(dev, sizeof(long long) * n);
    dist     = dbuf(dev, sizeof(float) * n);
    dist_alt = dbuf(dev, sizeof(float) * n);
    rows     = dbuf(dev, sizeof(int32_t) * n);
    rows_alt = dbuf(dev, sizeof(int32_t) * n);
    ukey     = dbuf(dev, sizeof(long long) * n);
    pop      = dbuf(dev, sizeof(int32_t) * n);
    start    = dbuf(dev, sizeof(int32_t) * n);
    keep     = dbuf(dev, sizeof(int32_t) * n);
    slot     = dbuf(dev, sizeof(int32_t) * n);
    key      = dbuf(dev, sizeof(long long) * n);
    kstart   = dbuf(dev, sizeof(int32_t) * n);
    kpop     = dbuf(dev, sizeof(int32_t) * n);
    bucket   = dbuf(dev, sizeof(int32_t) * n);
    bucket_alt = dbuf(dev, sizeof(int32_t) * n);
    perm     = dbuf(dev, sizeof(int32_t) * n);
    perm_alt = dbuf(dev, sizeof(int32_t) * n);
    skeys    = dbuf(dev, sizeof(long long) * n);
    runs     = dbuf(dev, sizeof(int64_t));
    lists    = dbuf(dev, sizeof(int32_t) * n * l);
    offsets  = dbuf(dev, sizeof(int32_t) * T1);
    size_t a = 0, b = 0, c = 0, d = 0, e = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, a, dist.as<unsigned>(), dist_alt.as<unsigned>(), rows.as<int32_t>(),
                                    rows_alt.as<int32_t>(), n);
    cub::DeviceRadixSort::SortPairs(nullptr, b, code.as<long long>(), code_alt.as<long long>(), rows.as<int32_t>(),
                                    rows_alt.as<int32_t>(), n);
    cub::DeviceRunLengthEncode::Encode(nullptr, c, code.as<long long>(), ukey.as<long long>(), pop.as<int32_t>(),
                                       runs.as<int64_t>(), n);
    cub::DeviceScan::ExclusiveSum(nullptr, d, pop.as<int32_t>(), start.as<int32_t>(), n);
    cub::DeviceRadixSort::SortPairs(nullptr, e, bucket.as<int32_t>(), bucket_alt.as<int32_t>(), perm.as<int32_t>(),
                                    perm_alt.as<int32_t>(), n);
    tmp_bytes = std::max({a, b, c, d, e});
    tmp       = dbuf(dev, tmp_bytes);
  }
};

template <int B>
void cells_of_copy(cell_scratch& sc, const __half* x, const float* mean, const float* proj_c, const float* shift_c,
                   int64_t n, int D, index_params const& params, copy_cells& out, cudaStream_t s)
{
  const int w = 8 * B, l = params.list_len;
  const int L = static_cast<int>(params.spacings.size());
  const int64_t T = int64_t{1} << params.log_buckets, T1 = T + 1;
  rows_times(x, mean, proj_c, shift_c, n, D, w, sc.y.as<float>(), s);
  int64_t row = 0;
  for (int j = 0; j < L; j++) {
    const float f     = params.spacings[j];
    const float inv_f = static_cast<float>(1.0 / static_cast<double>(f));
    cell_of_rows_kernel<B><<<grid_for(n, 128), 128, 0, s>>>(sc.y.as<float>(), n, f, inv_f, sc.code.as<long long>(),
                                                             sc.dist.as<float>());
    iota_kernel<<<grid_for(n, 256), 256, 0, s>>>(sc.rows.as<int32_t>(), n);
    // rows by distance to their own cell centre (non-negative floats order as their bit patterns) ...
    size_t tb = sc.tmp_bytes;
    cub::DeviceRadixSort::SortPairs(sc.tmp.ptr, tb, sc.dist.as<unsigned>(), sc.dist_alt.as<unsigned>(),
                                    sc.rows.as<int32_t>(), sc.rows_alt.as<int32_t>(), n, 0, 32, s);
    // ... then, keeping that order inside a cell, by cell code: the runs are the cells
    gather_kernel<long long><<<grid_for(n, 256), 256, 0, s>>>(sc.code.as<long long>(), sc.rows_alt.as<int32_t>(), n,
                                                             sc.code_alt.as<long long>());
    tb = sc.tmp_bytes;
    cub::DeviceRadixSort::SortPairs(sc.tmp.ptr, tb, sc.code_alt.as<long long>(), sc.code.as<long long>(),
                                    sc.rows_alt.as<int32_t>(), sc.rows.as<int32_t>(), n, 0, 64, s);
    tb = sc.tmp_bytes;
    cub::DeviceRunLengthEncode::Encode(sc.tmp.ptr, tb, sc.code.as<long long>(), sc.ukey.as<long long>(),
                                       sc.pop.as<int32_t>(), sc.runs.as<int64_t>(), n, s);
    int64_t runs = 0;
    OCTEX_CUDA_TRY(cudaMemcpyAsync(&runs, sc.runs.ptr, sizeof(runs), cudaMemcpyDeviceToHost, s));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    tb = sc.tmp_bytes;
    cub::DeviceScan::ExclusiveSum(sc.tmp.ptr, tb, sc.pop.as<int32_t>(), sc.start.as<int32_t>(), runs, s);
    // the kept cells: all at the coarsest spacing, else those of at least min_cell rows
    const bool filter = params.min_cell > 1 && j < L - 1;
    OCTEX_EXPECTS(runs > 0, "octex: a spacing of a copy produced no cell at all");
    keep_kernel<<<grid_for(runs, 256), 256, 0, s>>>(sc.pop.as<int32_t>(), runs, filter ? params.min_cell : 0,
                                                    sc.keep.as<int32_t>());
    tb = sc.tmp_bytes;
    cub::DeviceScan::ExclusiveSum(sc.tmp.ptr, tb, sc.keep.as<int32_t>(), sc.slot.as<int32_t>(), runs, s);
    int32_t last_slot = 0, last_keep = 0;
    if (runs > 0) {
      OCTEX_CUDA_TRY(cudaMemcpyAsync(&last_slot, sc.slot.as<int32_t>() + runs - 1, 4, cudaMemcpyDeviceToHost, s));
      OCTEX_CUDA_TRY(cudaMemcpyAsync(&last_keep, sc.keep.as<int32_t>() + runs - 1, 4, cudaMemcpyDeviceToHost, s));
      OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    }
    const int64_t cells = static_cast<int64_t>(last_slot) + last_keep;
    if (runs > 0)
      compact_cells_kernel<<<grid_for(runs, 256), 256, 0, s>>>(
      sc.ukey.as<long long>(), sc.start.as<int32_t>(), sc.pop.as<int32_t>(), sc.keep.as<int32_t>(),
      sc.slot.as<int32_t>(), runs, sc.key.as<long long>(), sc.kstart.as<int32_t>(), sc.kpop.as<int32_t>());
    // (bucket, code) order of the cells and the bucket bounds (build_cells.cuh:387-449): the cells
    // are in code order already and the sort by bucket is stable
    if (cells > 0) {
      bucket_kernel<<<grid_for(cells, 256), 256, 0, s>>>(sc.key.as<long long>(), cells, T - 1, sc.bucket.as<int32_t>());
      iota_kernel<<<grid_for(cells, 256), 256, 0, s>>>(sc.perm.as<int32_t>(), cells);
      tb = sc.tmp_bytes;
      cub::DeviceRadixSort::SortPairs(sc.tmp.ptr, tb, sc.bucket.as<int32_t>(), sc.bucket_alt.as<int32_t>(),
                                      sc.perm.as<int32_t>(), sc.perm_alt.as<int32_t>(), cells, 0, params.log_buckets, s);
      gather_kernel<long long><<<grid_for(cells, 256), 256, 0, s>>>(sc.key.as<long long>(), sc.perm_alt.as<int32_t>(),
                                                                   cells, sc.skeys.as<long long>());
      cell_lists_kernel<<<grid_for(cells * l, 256), 256, 0, s>>>(sc.rows.as<int32_t>(), sc.kstart.as<int32_t>(),
                                                                 sc.kpop.as<int32_t>(), sc.perm_alt.as<int32_t>(), cells,
                                                                 l, sc.lists.as<int32_t>());
    }
    bucket_bounds_kernel<<<grid_for(T1, 256), 256, 0, s>>>(sc.bucket_alt.as<int32_t>(), cells, T1,
                                                           sc.offsets.as<int32_t>());
    OCTEX_CUDA_TRY(cudaPeekAtLastError());
    const size_t l0 = out.lists.size(), k0 = out.keys.size(), o0 = out.offsets.size();
    out.lists.resize(l0 + static_cast<size_t>(cells) * l);
    out.keys.resize(k0 + static_cast<size_t>(cells));
    out.offsets.resize(o0 + static_cast<size_t>(T1));
    if (cells > 0) {
      OCTEX_CUDA_TRY(cudaMemcpyAsync(out.lists.data() + l0, sc.lists.ptr, sizeof(int32_t) * cells * l,
                                     cudaMemcpyDeviceToHost, s));
      OCTEX_CUDA_TRY(cudaMemcpyAsync(out.keys.data() + k0, sc.skeys.ptr, sizeof(int64_t) * cells,
                                     cudaMemcpyDeviceToHost, s));
    }
    OCTEX_CUDA_TRY(cudaMemcpyAsync(out.offsets.data() + o0, sc.offsets.ptr, sizeof(int32_t) * T1,
                                   cudaMemcpyDeviceToHost, s));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    out.base.push_back(static_cast<int32_t>(row));
    out.cells.push_back(cells);
    row += cells;
  }
}

// ---- int8 sketch (build_setup.cuh:177-264) --------------------------------------------------------

__global__ void amax_kernel(const float* __restrict__ v, int64_t n, int S, unsigned* __restrict__ amax)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n * S) atomicMax(amax + i % S, __float_as_uint(fabsf(v[i])));
}

__global__ void quantize_kernel(const float* __restrict__ v, const float* __restrict__ scale, int64_t n, int S,
                                signed char* __restrict__ out)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n * S) return;
  const float q = rintf(__fdiv_rn(v[i], scale[i % S]));
  out[i]        = static_cast<signed char>(fminf(127.f, fmaxf(-127.f, q)));
}

// ---- exact neighbor table (build_table.cuh:60-142) ------------------------------------------------

__global__ void row_norms_kernel(const __half* __restrict__ x, int64_t n, int D, float* __restrict__ norm)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int k = 0; k < D; k++) {
    const float v = __half2float(x[i * D + k]);
    acc           = __fmaf_rn(v, v, acc);
  }
  norm[i] = acc;
}

// The K nearest rows of every row by squared distance |a|^2 + |b|^2 - 2 a.b, the dot products of
// fp16 rows accumulated in fp32. A block owns 128 query rows and walks over all rows in tiles of
// 128: the 128 x 128 dot products of a tile are made by 256 threads (8 x 8 each) from operands
// staged in shared memory, the squared distances are left in shared memory, and one thread per
// query row scans its 128 of them against the K-th best it has so far, inserting the few that
// beat it into its sorted list in global memory (by the time a few tiles have passed, almost none
// does: a row meets about K (1 + ln(n / K)) improvements in all).
constexpr int kKnnTile = 128, kKnnDim = 16;
__global__ void __launch_bounds__(256)
  knn_kernel(const __half* __restrict__ x, const float* __restrict__ norm, int64_t n, int D, int K,
             int64_t q_first, int64_t q_count, int32_t* __restrict__ best_id, float* __restrict__ best_d)
{
  extern __shared__ __align__(16) unsigned char knn_smem[];
  float(*qs)[kKnnTile + 4] = reinterpret_cast<float(*)[kKnnTile + 4]>(knn_smem);  // [kKnnDim][128]
  float(*rs)[kKnnTile + 4] = qs + kKnnDim;                                        // [kKnnDim][128]
  float(*dt)[kKnnTile + 1] = reinterpret_cast<float(*)[kKnnTile + 1]>(rs + kKnnDim);  // [128][128]
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int64_t q0 = q_first + static_cast<int64_t>(blockIdx.x) * kKnnTile;
  int32_t* my_id = nullptr;
  float* my_d    = nullptr;
  float kth      = INFINITY;
  int have       = 0;
  if (threadIdx.x < kKnnTile && q0 + threadIdx.x < q_first + q_count) {
    my_id = best_id + (q0 - q_first + threadIdx.x) * K;
    my_d  = best_d + (q0 - q_first + threadIdx.x) * K;
  }
  for (int64_t r0 = 0; r0 < n; r0 += kKnnTile) {
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; a++)
#pragma unroll
      for (int b = 0; b < 8; b++)
        acc[a][b] = 0.f;
    for (int d0 = 0; d0 < D; d0 += kKnnDim) {
      for (int t = threadIdx.x; t < kKnnTile * kKnnDim; t += 256) {
        const int r = t / kKnnDim, d = t % kKnnDim;
        qs[d][r] = (q0 + r < n && d0 + d < D) ? __half2float(x[(q0 + r) * D + d0 + d]) : 0.f;
        rs[d][r] = (r0 + r < n && d0 + d < D) ? __half2float(x[(r0 + r) * D + d0 + d]) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int d = 0; d < kKnnDim; d++) {
        float a[8], b[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
          a[u] = qs[d][ty * 8 + u];
          b[u] = rs[d][tx * 8 + u];
        }
#pragma unroll
        for (int u = 0; u < 8; u++)
#pragma unroll
          for (int v = 0; v < 8; v++)
            acc[u][v] = __fmaf_rn(a[u], b[v], acc[u][v]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int64_t q = q0 + ty * 8 + u;
      const float qn  = q < n ? norm[q] : 0.f;
#pragma unroll
      for (int v = 0; v < 8; v++) {
        const int64_t r = r0 + tx * 8 + v;
        float d2        = INFINITY;
        if (q < n && r < n && r != q) d2 = fmaxf(__fadd_rn(__fadd_rn(qn, norm[r]), -2.f * acc[u][v]), 0.f);
        dt[ty * 8 + u][tx * 8 + v] = d2;
      }
    }
    __syncthreads();
    if (my_id != nullptr) {
      for (int c = 0; c < kKnnTile; c++) {
        const float d2 = dt[threadIdx.x][c];
        if (!(d2 < kth)) continue;
        // sorted insertion (ascending distance; equal distances keep the earlier row first)
        int at = have < K ? have : K - 1;
        while (at > 0 && my_d[at - 1] > d2) {
          my_d[at]  = my_d[at - 1];
          my_id[at] = my_id[at - 1];
          at--;
        }
        my_d[at]  = d2;
        my_id[at] = static_cast<int32_t>(r0 + c);
        if (have < K) have++;
        if (have == K) kth = my_d[K - 1];
      }
    }
    __syncthreads();
  }
  if (my_id != nullptr)
    for (int t = have; t < K; t++) {
      my_id[t] = -1;
      my_d[t]  = INFINITY;
    }
}

// Reverse edges (build_table.cuh:171-251): row v names u among its first h neighbors -> u may list
// v. One entry per such pair, keyed (u, distance) so that a sort brings the nearest proposers of
// every u together.
__global__ void reverse_edges_kernel(const int32_t* __restrict__ fwd, const float* __restrict__ fd, int64_t n, int K,
                                     int h, unsigned long long* __restrict__ key, int32_t* __restrict__ src)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n * h) return;
  const int64_t v = i / h;
  const int t     = static_cast<int>(i % h);
  const int32_t u = fwd[v * K + t];
  key[i] = u < 0 ? ~0ULL : (static_cast<unsigned long long>(static_cast<unsigned>(u)) << 32) | __float_as_uint(fd[v * K + t]);
  src[i] = static_cast<int32_t>(v);
}

// first[u] = position of the first sorted reverse edge whose target is >= u, u = 0 .. n
__global__ void edge_bounds_kernel(const unsigned long long* __restrict__ key, int64_t edges, int64_t n,
                                   int64_t* __restrict__ first)
{
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (u > n) return;
  int64_t lo = 0, hi = edges;
  const unsigned long long want = static_cast<unsigned long long>(u) << 32;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (key[mid] < want)
      lo = mid + 1;
    else
      hi = mid;
  }
  first[u] = lo;
}

// The reverse-edge rule (build_table.cuh:163-251,529-554): a row's table is its first kf forward
// neighbors, then up to kr nearest reverse edges, then the remaining of its K forward ones;
// duplicates dropped (the first occurrence stays), the first k kept, ordered nearest first (equal
// distances by id). The exact table takes K = k, kf = kr = k / 2 (the half rule), the searched one
// K = 3k / 2, kf = k / 4, kr = 3k / 4. One warp per row; the candidates (at most K + kr <= 256)
// sit in shared memory.
constexpr int kMergeMax = 256;
__global__ void __launch_bounds__(128)
  half_rule_kernel(const int32_t* __restrict__ fwd, const float* __restrict__ fd, int K,
                   const unsigned long long* __restrict__ ekey, const int32_t* __restrict__ esrc,
                   const int64_t* __restrict__ efirst, int64_t n, int k, int kf, int kr, int32_t* __restrict__ table)
{
  __shared__ int32_t cid[4][kMergeMax];
  __shared__ float cd[4][kMergeMax];
  __shared__ unsigned char ok[4][kMergeMax];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t v = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (v >= n) return;
  const int64_t e0 = efirst[v], e1 = efirst[v + 1];
  const int nrev   = static_cast<int>(min(e1 - e0, static_cast<int64_t>(kr)));
  const int total  = K + nrev;  // all K forward neighbors (self already dropped) and the reverse ones
  for (int t = lane; t < total; t += 32) {
    int32_t id;
    float d;
    if (t < kf) {
      id = fwd[v * K + t];
      d  = fd[v * K + t];
    } else if (t < kf + nrev) {
      id = esrc[e0 + (t - kf)];
      d  = __uint_as_float(static_cast<unsigned>(ekey[e0 + (t - kf)] & 0xffffffffULL));
    } else {
      id = fwd[v * K + (t - nrev)];
      d  = fd[v * K + (t - nrev)];
    }
    cid[warp][t] = id;
    cd[warp][t]  = d;
  }
  __syncwarp();
  // keep the first occurrence of every id, in priority order; then the first k of those
  for (int t = lane; t < total; t += 32) {
    const int32_t id = cid[warp][t];
    bool keep        = id >= 0;
    for (int s = 0; s < t && keep; s++)
      keep = cid[warp][s] != id;
    ok[warp][t] = keep ? 1 : 0;
  }
  __syncwarp();
  if (lane == 0) {
    int taken = 0;
    for (int t = 0; t < total; t++) {
      if (ok[warp][t] && taken < k)
        taken++;
      else
        ok[warp][t] = 0;
    }
  }
  __syncwarp();
  // rank of every kept candidate by (distance, id) among the kept ones = its column
  for (int t = lane; t < total; t += 32) {
    if (!ok[warp][t]) continue;
    const float d    = cd[warp][t];
    const int32_t id = cid[warp][t];
    int rank         = 0;
    for (int s = 0; s < total; s++)
      if (ok[warp][s] && (cd[warp][s] < d || (cd[warp][s] == d && cid[warp][s] < id))) rank++;
    table[v * k + rank] = id;
  }
  __syncwarp();
  int kept = 0;
  for (int t = lane; t < total; t += 32)
    kept += ok[warp][t];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    kept += __shfl_xor_sync(0xffffffffu, kept, o);
  for (int t = kept + lane; t < k; t += 32)
    table[v * k + t] = -1;
}

}  // namespace

void exact_neighbors(const __half* x, int64_t n, int D, int K, int method, int32_t* ids, float* dist, cudaStream_t s)
{
  OCTEX_EXPECTS(n > 0 && D > 0 && K > 0, "octex: exact_neighbors needs rows, a dimension and K >= 1");
  OCTEX_EXPECTS(method >= 0 && method <= 2, "octex: exact_neighbors method is 0 (choose), 1 (tensor cores) or 2 (plain)");
  int dev = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&dev));
  dbuf norm(dev, sizeof(float) * n);
  row_norms_kernel<<<grid_for(n, 128), 128, 0, s>>>(x, n, D, norm.as<float>());
  const bool covered = kernels::knn_tc_supported(n, D, K);
  OCTEX_EXPECTS(method != 1 || covered,
                "octex: the tensor-core neighbor scan needs a dimension that is a multiple of 8 and K <= 120");
  if (method == 1 || (method == 0 && covered)) {
    dbuf error(dev, sizeof(int));
    OCTEX_CUDA_TRY(cudaMemsetAsync(error.ptr, 0, sizeof(int), s));
    kernels::knn_tc(x, norm.as<float>(), n, D, K, 0, n, ids, dist, error.as<int>(), s);
    OCTEX_CUDA_TRY(cudaPeekAtLastError());
    const int gave_up = to_host<int>(error.ptr, 1)[0];
    OCTEX_EXPECTS(gave_up == 0, "octex: the neighbor scan gave up waiting inside the kernel (code " +
                                  std::to_string(gave_up) + "); its lists are incomplete");
  } else {
    const size_t smem = sizeof(float) * (2 * kKnnDim * (kKnnTile + 4) + kKnnTile * (kKnnTile + 1));
    OCTEX_CUDA_TRY(cudaFuncSetAttribute(knn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    knn_kernel<<<grid_for(n, kKnnTile), 256, smem, s>>>(x, norm.as<float>(), n, D, K, 0, n, ids, dist);
    OCTEX_CUDA_TRY(cudaPeekAtLastError());
  }
  OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
}

namespace {

// Reverse-edge merge of forward rows fwd / fd [n, K] (nearest first, -1 padded) into table rows
// out [n, k]: every row v proposes itself to the rows among its first ks neighbors, a row takes its
// first kf forward neighbors, up to kr nearest proposers, then its other forward neighbors
// (half_rule_kernel). All pointers are device memory of `dev`.
void reverse_merge(int dev, const int32_t* fwd, const float* fd, int64_t n, int K, int ks, int kf, int kr, int k,
                   int32_t* out, cudaStream_t s)
{
  OCTEX_EXPECTS(K + kr <= kMergeMax && ks <= K && kf <= K && k <= K + kr, "octex: reverse merge: rows too long");
  const int64_t edges = n * ks;
  dbuf ekey(dev, 8 * edges), ekey_s(dev, 8 * edges), esrc(dev, 4 * edges), esrc_s(dev, 4 * edges),
    efirst(dev, 8 * (n + 1));
  reverse_edges_kernel<<<grid_for(edges, 256), 256, 0, s>>>(fwd, fd, n, K, ks, ekey.as<unsigned long long>(),
                                                            esrc.as<int32_t>());
  size_t tb = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, tb, ekey.as<unsigned long long>(), ekey_s.as<unsigned long long>(),
                                  esrc.as<int32_t>(), esrc_s.as<int32_t>(), edges);
  dbuf tmp(dev, tb);
  cub::DeviceRadixSort::SortPairs(tmp.ptr, tb, ekey.as<unsigned long long>(), ekey_s.as<unsigned long long>(),
                                  esrc.as<int32_t>(), esrc_s.as<int32_t>(), edges, 0, 64, s);
  edge_bounds_kernel<<<grid_for(n + 1, 256), 256, 0, s>>>(ekey_s.as<unsigned long long>(), edges, n,
                                                          efirst.as<int64_t>());
  half_rule_kernel<<<grid_for(n, 4), 128, 0, s>>>(fwd, fd, K, ekey_s.as<unsigned long long>(), esrc_s.as<int32_t>(),
                                                  efirst.as<int64_t>(), n, k, kf, kr, out);
  OCTEX_CUDA_TRY(cudaPeekAtLastError());
  OCTEX_CUDA_TRY(cudaStreamSynchronize(s));  // the scratch arrays go with this scope
}

// ---- the directory ---------------------------------------------------------------------------------

/// A .npy file (format 1.0, little endian, C order, header padded to 64 bytes) written in pieces.
class npy_writer {
 public:
  npy_writer(std::string const& path, const char* descr, std::vector<int64_t> const& shape)
    : out_(path, std::ios::binary | std::ios::trunc), path_(path)
  {
    OCTEX_EXPECTS(out_.good(), "octex: cannot write " + path);
    std::ostringstream dict;
    dict << "{'descr': '" << descr << "', 'fortran_order': False, 'shape': (";
    for (size_t i = 0; i < shape.size(); i++)
      dict << shape[i] << (shape.size() == 1 || i + 1 < shape.size() ? "," : "") << (i + 1 < shape.size() ? " " : "");
    dict << "), }";
    std::string h = dict.str();
    const size_t unpadded = 10 + h.size() + 1;
    h.append((64 - unpadded % 64) % 64, ' ');
    h.push_back('\n');
    const unsigned char magic[8] = {0x93, 'N', 'U', 'M', 'P', 'Y', 1, 0};
    out_.write(reinterpret_cast<const char*>(magic), 8);
    const uint16_t len = static_cast<uint16_t>(h.size());
    out_.write(reinterpret_cast<const char*>(&len), 2);
    out_.write(h.data(), static_cast<std::streamsize>(h.size()));
  }
  void write(const void* data, size_t bytes) { out_.write(static_cast<const char*>(data), static_cast<std::streamsize>(bytes)); }
  void zeros(size_t bytes)
  {
    static const std::vector<char> z(1 << 20, 0);
    while (bytes > 0) {
      const size_t nb = std::min(bytes, z.size());
      out_.write(z.data(), static_cast<std::streamsize>(nb));
      bytes -= nb;
    }
  }
  void close()
  {
    out_.flush();
    OCTEX_EXPECTS(out_.good(), "octex: writing " + path_ + " failed");
    out_.close();
  }

 private:
  std::ofstream out_;
  std::string path_;
};

template <typename T>
void write_array(std::string const& path, const char* descr, std::vector<int64_t> const& shape, const T* data)
{
  size_t count = 1;
  for (auto v : shape)
    count *= static_cast<size_t>(v);
  npy_writer w(path, descr, shape);
  w.write(data, count * sizeof(T));
  w.close();
}

auto seconds_since(std::chrono::steady_clock::time_point t0) -> double
{
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

}  // namespace

auto auto_sketch_width(int64_t dim) -> int
{
  // build.cu:118-121 of the reference
  return static_cast<int>(std::max<int64_t>(std::min<int64_t>(dim / 16 * 16, 128), std::min<int64_t>(dim, 16)));
}

namespace {

__global__ void rows_to_float_kernel(const __half* __restrict__ x, int64_t count, float* __restrict__ q)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) q[i] = __half2float(x[i]);
}

// The answers of a search of base rows [r0, r0 + m) for kq neighbors each, as forward rows of kin:
// the row itself is dropped where it was found (else the last answer is).
__global__ void forward_rows_kernel(const long long* __restrict__ ids, const float* __restrict__ dist, int64_t r0,
                                    int64_t m, int kq, int kin, int32_t* __restrict__ fwd, float* __restrict__ fd)
{
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= m) return;
  int out = 0;
  for (int t = 0; t < kq && out < kin; t++) {
    const long long id = ids[r * kq + t];
    if (id == r0 + r) continue;
    fwd[(r0 + r) * kin + out] = id < 0 ? -1 : static_cast<int32_t>(id);
    fd[(r0 + r) * kin + out]  = id < 0 ? INFINITY : dist[r * kq + t];
    out++;
  }
  for (; out < kin; out++) {
    fwd[(r0 + r) * kin + out] = -1;
    fd[(r0 + r) * kin + out]  = INFINITY;
  }
}

}  // namespace

void searched_table(resources const& res, index& idx, int k, int passes, bool reverse_edges, bool sketch_order,
                    int32_t* table_host, bool verbose)
{
  auto& ix = idx.impl();
  auto& p  = ix.part;
  OCTEX_EXPECTS(ix.world == 1, "octex: the searched table is made by one process");
  OCTEX_EXPECTS(!p.vectors.host && !p.vector_rows.on, "octex: the searched table reads the fp16 rows from this GPU");
  const int64_t n = ix.n;
  const int D     = static_cast<int>(ix.dim);
  // rows, passes and rule of build_table.cuh:586-614: forward rows of 3k/2 from a search for one
  // more; a first round only, then 2 and 3 waves over the merged table of the pass before; a merged
  // row keeps k/4 forward entries first and up to 3k/4 reverse ones
  const int kin = k + k / 2, kq = kin + 1, kf = std::max(1, k / 4), kr = std::max(1, k - kf);
  OCTEX_EXPECTS(k >= 1 && kq < n, "octex: table_len too large for the dataset");
  OCTEX_EXPECTS(kq <= kernels::kMaxRerank, "octex: table_len too large for the searched table");
  passes = std::clamp(passes, 1, 3);
  const int pass_waves[3] = {0, 2, 3}, pass_starts[3] = {64, 128, 128};
  int cur = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  cudaStream_t s = res.stream;
  const int64_t chunk = std::min<int64_t>(n, 100000);
  dbuf q(p.device, sizeof(float) * chunk * D), ids(p.device, sizeof(long long) * chunk * kq),
    dist(p.device, sizeof(float) * chunk * kq), fwd(p.device, sizeof(int32_t) * n * kin),
    fd(p.device, sizeof(float) * n * kin), merged(p.device, sizeof(int32_t) * n * k);
  for (int v = 0; v < passes; v++) {
    const auto t0 = std::chrono::steady_clock::now();
    search_params sp;
    sp.read         = std::min(64, ix.list_len);
    sp.starts       = std::max(pass_starts[v], kq);
    sp.waves        = ix.table_len > 0 ? pass_waves[v] : 0;
    sp.batch        = 10000;
    sp.sketch_rank  = true;
    sp.final_rerank = sketch_order ? 0 : kq;  // table_sketch_order: no exact rerank of the answers
    for (int64_t r0 = 0; r0 < n; r0 += chunk) {
      const int64_t m = std::min(chunk, n - r0);
      OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));  // the rows' owner stream, before this one reads them
      rows_to_float_kernel<<<grid_for(m * D, 256), 256, 0, s>>>(p.vectors.as<__half>() + r0 * D, m * D, q.as<float>());
      detail::search_impl(res, sp, idx, q.as<float>(), m, D, reinterpret_cast<int64_t*>(ids.ptr), dist.as<float>(), kq, false, false);
      forward_rows_kernel<<<grid_for(m, 128), 128, 0, s>>>(ids.as<long long>(), dist.as<float>(), r0, m, kq, kin,
                                                          fwd.as<int32_t>(), fd.as<float>());
      OCTEX_CUDA_TRY(cudaPeekAtLastError());
    }
    OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    if (reverse_edges) {
      reverse_merge(p.device, fwd.as<int32_t>(), fd.as<float>(), n, kin, kin, kf, kr, k, merged.as<int32_t>(), s);
    } else {
      OCTEX_CUDA_TRY(cudaMemcpy2DAsync(merged.ptr, sizeof(int32_t) * k, fwd.ptr, sizeof(int32_t) * kin, sizeof(int32_t) * k,
                                       n, cudaMemcpyDeviceToDevice, s));
      OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    }
    detail::set_table(ix, merged.as<int32_t>(), k);
    if (verbose)
      std::fprintf(stderr, "octex: searched table, pass %d of %d (%d waves, %d starts): %.2f s\n", v + 1, passes,
                   sp.waves, sp.starts, seconds_since(t0));
  }
  if (table_host != nullptr)
    OCTEX_CUDA_TRY(cudaMemcpy(table_host, merged.ptr, merged.size, cudaMemcpyDeviceToHost));
  OCTEX_CUDA_TRY(cudaSetDevice(cur));
}

void build(resources const& res, index_params const& given, build_dataset const& data, std::string const& path)
{
  index_params params = given;
  if (params.spacings.empty()) params.spacings = {2.0f, 2.5f, 3.2f, 4.0f, 5.0f};
  const int64_t n = data.rows, D64 = data.dim;
  OCTEX_EXPECTS(data.data != nullptr && n >= 2 && D64 >= 2, "octex: the dataset is empty");
  OCTEX_EXPECTS(D64 % 2 == 0, "octex: the dimension must be even");
  OCTEX_EXPECTS(n < (int64_t{1} << 31), "octex: this builder takes fewer than 2^31 rows");
  OCTEX_EXPECTS((params.blocks >= 1 && params.blocks <= 6) || params.blocks == 8, "octex: blocks must be 1-6 or 8");
  OCTEX_EXPECTS(params.copies >= 1 && params.list_len >= 1, "octex: copies and list_len must be positive");
  OCTEX_EXPECTS(params.log_buckets >= 1 && params.log_buckets <= 30, "octex: log_buckets in [1, 30]");
  OCTEX_EXPECTS(!params.spacings.empty() && params.spacings.size() <= 16, "octex: 1 to 16 spacings");
  OCTEX_EXPECTS(params.table_len >= 0 && params.table_len < n && params.table_len + params.table_len / 2 <= kMergeMax,
                "octex: table_len must be in [0, n) and at most 170");
  const int D = static_cast<int>(D64), w = 8 * params.blocks, L = static_cast<int>(params.spacings.size());
  const int S = params.sketch_width > 0 ? static_cast<int>(std::min<int64_t>(params.sketch_width, D)) : auto_sketch_width(D);
  OCTEX_EXPECTS(S % 16 == 0 && S <= 512, "octex: sketch width: a multiple of 16, <= 512");
  const int p = static_cast<int>(std::min<int64_t>(params.pca_dims, D));
  const int64_t T1 = (int64_t{1} << params.log_buckets) + 1;
  cudaStream_t s = res.stream;
  int dev = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&dev));
  std::vector<std::pair<std::string, double>> took;
  auto t0 = std::chrono::steady_clock::now();

  // the dataset as fp16 on the GPU
  dbuf x16(dev, sizeof(__half) * n * D);
  if (data.f16) {
    OCTEX_CUDA_TRY(cudaMemcpyAsync(x16.ptr, data.data, x16.size, cudaMemcpyDefault, s));
  } else {
    const int64_t chunk = int64_t{1} << 26;  // elements
    dbuf stage(dev, sizeof(float) * std::min<int64_t>(chunk, n * D));
    for (int64_t e0 = 0; e0 < n * D; e0 += chunk) {
      const int64_t ne = std::min(chunk, n * D - e0);
      OCTEX_CUDA_TRY(cudaMemcpyAsync(stage.ptr, static_cast<const float*>(data.data) + e0, sizeof(float) * ne,
                                     cudaMemcpyDefault, s));
      f32_to_f16_kernel<<<grid_for(ne, 256), 256, 0, s>>>(stage.as<float>(), ne, x16.as<__half>() + e0);
      OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    }
  }
  OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
  took.emplace_back("dataset", seconds_since(t0));

  // sample PCA, projections
  t0 = std::chrono::steady_clock::now();
  pca_result pca = sample_pca(x16.as<__half>(), n, D, s);
  std::vector<float> proj, shift;
  make_projections(pca, D, p, w, params.copies, params.seed, proj, shift);
  dbuf mean(dev, sizeof(float) * D), proj_d(dev, sizeof(float) * D * w), shift_d(dev, sizeof(float) * w);
  OCTEX_CUDA_TRY(cudaMemcpyAsync(mean.ptr, pca.mean.data(), mean.size, cudaMemcpyHostToDevice, s));
  took.emplace_back("pca", seconds_since(t0));

  // cells of every copy
  t0 = std::chrono::steady_clock::now();
  std::vector<copy_cells> cc(params.copies);
  {
    cell_scratch sc(dev, n, w, params.list_len, T1);
    for (int c = 0; c < params.copies; c++) {
      OCTEX_CUDA_TRY(cudaMemcpyAsync(proj_d.ptr, proj.data() + static_cast<size_t>(c) * D * w, proj_d.size,
                                     cudaMemcpyHostToDevice, s));
      OCTEX_CUDA_TRY(cudaMemcpyAsync(shift_d.ptr, shift.data() + static_cast<size_t>(c) * w, shift_d.size,
                                     cudaMemcpyHostToDevice, s));
      switch (params.blocks) {
        case 1: cells_of_copy<1>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
        case 2: cells_of_copy<2>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
        case 3: cells_of_copy<3>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
        case 4: cells_of_copy<4>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
        case 5: cells_of_copy<5>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
        case 6: cells_of_copy<6>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
        default: cells_of_copy<8>(sc, x16.as<__half>(), mean.as<float>(), proj_d.as<float>(), shift_d.as<float>(), n, D, params, cc[c], s); break;
      }
      if (params.verbose && (c % 10 == 0 || c == params.copies - 1)) {
        std::fprintf(stderr, "  copy %d: cells per level", c);
        for (auto m : cc[c].cells)
          std::fprintf(stderr, " %lld", static_cast<long long>(m));
        std::fprintf(stderr, "\n");
      }
    }
  }
  took.emplace_back("cells", seconds_since(t0));

  // sketch
  t0 = std::chrono::steady_clock::now();
  std::vector<float> basis(static_cast<size_t>(D) * S), scale(S);
  for (int k = 0; k < D; k++)
    for (int c = 0; c < S; c++)
      basis[static_cast<size_t>(k) * S + c] = pca.vectors[static_cast<size_t>(k) * D + c];
  std::vector<int8_t> codes(static_cast<size_t>(n) * S);
  {
    const int64_t chunk = std::min<int64_t>(n, int64_t{1} << 18);
    dbuf basis_d(dev, sizeof(float) * D * S), v(dev, sizeof(float) * chunk * S), amax(dev, sizeof(unsigned) * S),
      scale_d(dev, sizeof(float) * S), q(dev, static_cast<size_t>(chunk) * S);
    OCTEX_CUDA_TRY(cudaMemcpyAsync(basis_d.ptr, basis.data(), basis_d.size, cudaMemcpyHostToDevice, s));
    OCTEX_CUDA_TRY(cudaMemsetAsync(amax.ptr, 0, amax.size, s));
    for (int64_t r0 = 0; r0 < n; r0 += chunk) {
      const int64_t m = std::min(chunk, n - r0);
      rows_times(x16.as<__half>() + r0 * D, mean.as<float>(), basis_d.as<float>(), nullptr, m, D, S, v.as<float>(), s);
      amax_kernel<<<grid_for(m * S, 256), 256, 0, s>>>(v.as<float>(), m, S, amax.as<unsigned>());
    }
    auto ha = to_host<unsigned>(amax.ptr, S);
    for (int k = 0; k < S; k++) {
      float am;
      std::memcpy(&am, &ha[k], sizeof(float));
      scale[k] = am > 0.f ? am / 127.f : 1.f;
    }
    OCTEX_CUDA_TRY(cudaMemcpyAsync(scale_d.ptr, scale.data(), scale_d.size, cudaMemcpyHostToDevice, s));
    for (int64_t r0 = 0; r0 < n; r0 += chunk) {
      const int64_t m = std::min(chunk, n - r0);
      rows_times(x16.as<__half>() + r0 * D, mean.as<float>(), basis_d.as<float>(), nullptr, m, D, S, v.as<float>(), s);
      quantize_kernel<<<grid_for(m * S, 256), 256, 0, s>>>(v.as<float>(), scale_d.as<float>(), m, S, q.as<signed char>());
      OCTEX_CUDA_TRY(cudaMemcpyAsync(codes.data() + r0 * S, q.ptr, static_cast<size_t>(m) * S, cudaMemcpyDeviceToHost, s));
      OCTEX_CUDA_TRY(cudaStreamSynchronize(s));
    }
  }
  took.emplace_back("sketch", seconds_since(t0));

  // neighbor table
  t0 = std::chrono::steady_clock::now();
  std::vector<int32_t> table;
  const int k = params.table_len;
  // above exact_table_max rows the table comes from the index's own search, once the rest of the
  // directory is there (build_table.cuh:729-790)
  const bool searched = k > 0 && n > params.exact_table_max;
  if (k > 0 && !searched) {
    const int K = k;  // self is excluded inside the scan
    dbuf fwd(dev, sizeof(int32_t) * n * K), fd(dev, sizeof(float) * n * K);
    exact_neighbors(x16.as<__half>(), n, D, K, 0, fwd.as<int32_t>(), fd.as<float>(), s);
    took.emplace_back("table_scan", seconds_since(t0));
    dbuf out(dev, sizeof(int32_t) * n * k);
    const int h = std::max(1, k / 2);
    if (params.reverse_edges) {
      reverse_merge(dev, fwd.as<int32_t>(), fd.as<float>(), n, K, h, h, h, k, out.as<int32_t>(), s);
      OCTEX_CUDA_TRY(cudaPeekAtLastError());
      table = to_host<int32_t>(out.ptr, static_cast<size_t>(n) * k);
    } else {
      table = to_host<int32_t>(fwd.ptr, static_cast<size_t>(n) * k);
    }
  }
  took.emplace_back("table", seconds_since(t0));

  // the directory; meta.json last: a directory without it is incomplete (build.cu:423-424)
  t0 = std::chrono::steady_clock::now();
  make_directory(path);
  const int C = params.copies;
  int64_t rows_max = 0, cells_max = 0;
  for (auto const& c : cc) {
    int64_t rows = 0;
    for (auto m : c.cells) {
      rows += m;
      cells_max = std::max(cells_max, m);
    }
    rows_max = std::max(rows_max, rows);
  }
  cells_max = std::max<int64_t>(cells_max, 1);
  const int64_t stride = std::max<int64_t>(rows_max, 1) * params.list_len;
  write_array(path + "/mean.npy", "<f4", {D}, pca.mean.data());
  write_array(path + "/proj.npy", "<f4", {C, D, w}, proj.data());
  write_array(path + "/shift.npy", "<f4", {C, w}, shift.data());
  {
    npy_writer lists(path + "/lists.npy", "<i4", {C, stride}), keys(path + "/keys.npy", "<i8", {C, L, cells_max}),
      offsets(path + "/offsets.npy", "<i4", {C, L, T1}), base(path + "/base.npy", "<i4", {C, L}),
      cells(path + "/cells.npy", "<i8", {C, L});
    for (auto const& c : cc) {
      lists.write(c.lists.data(), c.lists.size() * sizeof(int32_t));
      lists.zeros((static_cast<size_t>(stride) - c.lists.size()) * sizeof(int32_t));
      size_t at = 0;
      for (int j = 0; j < L; j++) {
        keys.write(c.keys.data() + at, static_cast<size_t>(c.cells[j]) * sizeof(int64_t));
        keys.zeros(static_cast<size_t>(cells_max - c.cells[j]) * sizeof(int64_t));
        at += static_cast<size_t>(c.cells[j]);
      }
      offsets.write(c.offsets.data(), c.offsets.size() * sizeof(int32_t));
      base.write(c.base.data(), c.base.size() * sizeof(int32_t));
      cells.write(c.cells.data(), c.cells.size() * sizeof(int64_t));
    }
    lists.close();
    keys.close();
    offsets.close();
    base.close();
    cells.close();
  }
  write_array(path + "/sketch_basis.npy", "<f4", {D, S}, basis.data());
  write_array(path + "/sketch_scale.npy", "<f4", {S}, scale.data());
  write_array(path + "/sketch.npy", "|i1", {n, S}, codes.data());
  {
    auto hx = to_host<uint16_t>(x16.ptr, static_cast<size_t>(n) * D);
    write_array(path + "/vectors.npy", "<f2", {n, D}, hx.data());
  }
  if (k > 0 && !searched) write_array(path + "/table.npy", "<i4", {n, k}, table.data());
  took.emplace_back("write", seconds_since(t0));
  auto write_meta = [&](int table_len) {
    std::ofstream meta(path + "/meta.json", std::ios::trunc);
    OCTEX_EXPECTS(meta.good(), "octex: cannot write " + path + "/meta.json");
    meta << "{\"format\": 1, \"n\": " << n << ", \"dim\": " << D << ", \"copies\": " << C << ", \"blocks\": "
         << params.blocks << ", \"spacings\": [";
    for (int j = 0; j < L; j++)
      meta << (j ? ", " : "") << params.spacings[j];
    meta << "], \"list_len\": " << params.list_len << ", \"log_buckets\": " << params.log_buckets
         << ", \"sketch_width\": " << S << ", \"table_len\": " << table_len << ", \"metric\": \"sqeuclidean\", \"build_seconds\": {";
    for (size_t i = 0; i < took.size(); i++)
      meta << (i ? ", " : "") << "\"" << took[i].first << "\": " << took[i].second;
    meta << "}}\n";
    meta.close();
    OCTEX_EXPECTS(meta.good(), "octex: writing " + path + "/meta.json failed");
  };
  if (!searched) {
    write_meta(k);
    return;
  }
  // the directory without a table is complete and loadable; the searched table is added to it
  write_meta(0);
  t0 = std::chrono::steady_clock::now();
  x16 = dbuf();  // the loaded index brings its own copy of the rows
  {
    load_params lp;
    lp.devices = {dev};
    lp.mode    = placement::replicate;
    index idx  = load(res, path, lp);
    table.assign(static_cast<size_t>(n) * k, -1);
    searched_table(res, idx, k, params.table_passes, params.reverse_edges, params.table_sketch_order, table.data(),
                   params.verbose);
  }
  write_array(path + "/table.npy", "<i4", {n, k}, table.data());
  took.emplace_back("table_searched", seconds_since(t0));
  write_meta(k);
}

}  // namespace octex_b200
