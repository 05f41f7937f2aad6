// TEST INFRASTRUCTURE ONLY. The reference's own search kernels
// (cpp/src/neighbors/octex/detail/search_kernels.cuh of hpdic/octex: probe_kernel, gather_kernel,
// rerank_keep_kernel, sketch_keep_kernel, pick_starts_kernel, final_rerank_kernel, take_k_kernel)
// compiled unmodified as device code and launched with the
// launch shapes of the reference's search.cu (:344-357, :393, :433-450, :453, :488), behind one
// host function with host pointers in and out. A GPU test feeds it the projected coordinates,
// sketch-space queries and queries of a batch and compares what the reference's kernels make of
// them — segments, candidate sets, sketch distances, kept lists — with the CPU checker, which is
// what pins the checker to the reference beyond the E8 decode. The header is included from where
// the reference sources lie; nothing of it is copied here. The only stand-in is a one-line
// raft/core/detail/macros.hpp (shim/) that defines RAFT_KERNEL.
#include "search_kernels.cuh"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

namespace ref = cuvs::neighbors::octex::detail;

namespace {

struct device_array {
  void* p = nullptr;
  cudaError_t err = cudaSuccess;
  device_array(const void* host, size_t bytes, bool copy = true)
  {
    err = cudaMalloc(&p, std::max<size_t>(bytes, 16));
    if (err == cudaSuccess && host != nullptr && copy && bytes != 0)
      err = cudaMemcpy(p, host, bytes, cudaMemcpyDefault);  // the source may be host or device memory
  }
  device_array(device_array const&) = delete;
  ~device_array() { cudaFree(p); }
  template <typename T>
  T* as() const
  {
    return static_cast<T*>(p);
  }
};

int log2_ceil(int64_t v)
{
  int e = 0;
  while ((int64_t{1} << e) < v)
    e++;
  return e;
}

int hash_log_for(int64_t entries)
{
  const int e = log2_ceil(static_cast<int64_t>(std::ceil(entries * ref::kHashGrow)));
  return std::clamp(e, ref::kMinLogHash, log2_ceil(ref::kMaxHash));
}

size_t gather_smem(int W, int sw, int C) { return static_cast<size_t>(W + 2 * sw + 2 * C + 1) * sizeof(int); }

}  // namespace

struct ref_search_args {
  // index (arrays of an index directory, host memory)
  int64_t n;
  int32_t dim, copies, blocks, levels, list_len, log_buckets, sketch_width, table_len;
  int64_t stride, mmax;
  const float* inv_f;         // [levels]
  const int32_t* lists;       // [copies, stride]
  const int64_t* keys;        // [copies, levels, mmax]
  const int32_t* offsets;     // [copies, levels, 2^log_buckets + 1]
  const int32_t* base;        // [copies, levels]
  const float* scale;         // [sketch_width]
  const int8_t* sketch;       // [n, sketch_width]
  const uint16_t* vectors;    // fp16 [n, dim]
  const int32_t* table;       // [n, table_len]
  // batch
  int32_t m;
  const uint16_t* y;          // fp16 [m, copies * 8 * blocks] projected coordinates
  const float* qs;            // [m, sketch_width]
  const float* q;             // [m, dim] uncentred queries
  // parameters
  int32_t read, starts, waves, rerank, wave_rerank, k;
  int32_t sketch_rank, final_rerank;  // rank by sketch distance; exact rerank of the first final_rerank kept
  // results
  int32_t* seg;               // [m, copies, 2]
  int32_t w1;                 // capacity of cand1 / dist1 per query (>= the hash set of round 1)
  int32_t* cand1;             // [m, w1]
  float* dist1;               // [m, w1]
  int32_t* n1;                // [m]
  int64_t* kept1_ids;         // [m, KO] after the first round
  float* kept1_dist;
  int64_t* kept_ids;          // [m, KO] after the waves
  float* kept_dist;
  int64_t* best_ids;          // [m, k] the search result (take_k or final_rerank)
  float* best_dist;
  float* kernel_ms;           // [2] (may be null): device time of the first round's kernels (lookup,
                              // gather, rerank) and of the waves' kernels, by CUDA events
  int32_t reps;               // > 1: the two stages run this many times and kernel_ms holds the medians
  int32_t flush_mb;           // > 0: a buffer of this many MB is overwritten before every timed stage,
                              // so that the stage starts with none of the index in the L2 cache
};

// Returns 0, a CUDA error code, or -1 for arguments the kernels cannot take.
extern "C" int ref_search_pipeline(const ref_search_args* a)
{
  const int m = a->m, C = a->copies, L = a->levels, S = a->sketch_width, D = a->dim;
  const int lr = std::min(a->read, a->list_len);
  const int KO = std::max(a->starts, a->k);
  const int64_t T1 = (int64_t{1} << a->log_buckets) + 1;
  if (a->blocks != 2 && a->blocks != 4) return -1;
  if (a->rerank > ref::kMaxRerank || a->wave_rerank > ref::kMaxRerank) return -1;
  const int FR = std::min(a->final_rerank, KO);
  if (a->sketch_rank && (KO > ref::kMaxSketchKO || (FR > 0 && (a->k > FR || FR > ref::kMaxRerank)))) return -1;
  if (a->k > KO) return -1;
  if (KO + std::max(a->rerank, a->wave_rerank) > ref::kMaxKeepSort) return -1;
  const int logW = hash_log_for(int64_t{C} * lr), W = 1 << logW;
  if (a->w1 < W) return -1;
  const int logW2 = hash_log_for(int64_t{a->starts} * a->table_len), W2 = 1 << logW2;
  const int width = 8 * a->blocks * C;

  device_array inv_f(a->inv_f, sizeof(float) * L), lists(a->lists, sizeof(int32_t) * C * a->stride),
    keys(a->keys, sizeof(int64_t) * C * L * a->mmax), offsets(a->offsets, sizeof(int32_t) * C * L * T1),
    base(a->base, sizeof(int32_t) * C * L), scale(a->scale, sizeof(float) * S),
    sketch(a->sketch, static_cast<size_t>(a->n) * S),
    vectors(a->vectors, sizeof(uint16_t) * a->n * D),
    table(a->table, sizeof(int32_t) * a->n * a->table_len), y(a->y, sizeof(uint16_t) * m * width),
    qs(a->qs, sizeof(float) * m * S), q(a->q, sizeof(float) * m * D);
  device_array seg(nullptr, sizeof(int2) * m * C), cand(nullptr, sizeof(int) * m * W),
    dist(nullptr, sizeof(float) * m * W), nin(nullptr, sizeof(int) * m),
    si(nullptr, sizeof(long long) * m * KO), sd(nullptr, sizeof(float) * m * KO),
    seg2(nullptr, sizeof(int2) * m * std::max(a->starts, 1)),
    cand2(nullptr, sizeof(int) * m * W2), dist2(nullptr, sizeof(float) * m * W2),
    n2(nullptr, sizeof(int) * m),
    done(nullptr, sizeof(long long) * m * std::max(a->starts * a->waves, 1)),
    bi(nullptr, sizeof(long long) * m * a->k), bd(nullptr, sizeof(float) * m * a->k);
  const long long xp = reinterpret_cast<long long>(vectors.p), tp = reinterpret_cast<long long>(table.p);
  device_array xptr(&xp, sizeof(xp)), tptr(&tp, sizeof(tp));
  for (const device_array* d : {&inv_f, &lists, &keys, &offsets, &base, &scale, &sketch, &vectors, &table,
                                &y, &qs, &q, &seg, &cand, &dist, &nin, &si, &sd, &seg2, &cand2, &dist2,
                                &n2, &done, &bi, &bd, &xptr, &tptr})
    if (d->err != cudaSuccess) return static_cast<int>(d->err);
  cudaMemset(cand.p, 0xff, sizeof(int) * m * W);
  cudaMemset(dist.p, 0, sizeof(float) * m * W);

  cudaEvent_t ev[4];
  for (auto& v : ev)
    cudaEventCreate(&v);
  const int reps = std::max(a->reps, 1);
  device_array flush(nullptr, a->flush_mb > 0 ? static_cast<size_t>(a->flush_mb) << 20 : 16);
  if (flush.err != cudaSuccess) return static_cast<int>(flush.err);
  auto flush_l2 = [&] {
    if (a->flush_mb > 0) cudaMemsetAsync(flush.p, 1, static_cast<size_t>(a->flush_mb) << 20);
  };
  cudaFuncSetAttribute(ref::gather_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(gather_smem(W, S, C)));
  if (a->waves > 0)
    cudaFuncSetAttribute(ref::gather_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(gather_smem(W2, S, a->starts)));
  std::vector<float> ms1, ms2;
  cudaError_t e = cudaSuccess;
  for (int rep = 0; rep < reps; rep++) {
    flush_l2();
    cudaEventRecord(ev[0]);
    // cell lookup (search.cu:105-137)
    {
      const int64_t tot = int64_t{m} * C;
      const unsigned grid = static_cast<unsigned>((tot + 255) / 256);
      if (a->blocks == 4)
        ref::probe_kernel<4><<<grid, 256>>>(y.as<__half>(), m, C, L, inv_f.as<float>(), offsets.as<int>(), T1,
                                            keys.as<long long>(), a->mmax, base.as<int>(), a->list_len, lr,
                                            a->log_buckets, seg.as<int2>());
      else
        ref::probe_kernel<2><<<grid, 256>>>(y.as<__half>(), m, C, L, inv_f.as<float>(), offsets.as<int>(), T1,
                                            keys.as<long long>(), a->mmax, base.as<int>(), a->list_len, lr,
                                            a->log_buckets, seg.as<int2>());
    }
    // first round: gather + sketch distances (search.cu:343-361), exact rerank into the kept list (:393)
    ref::gather_kernel<false><<<m, 256, gather_smem(W, S, C)>>>(
      seg.as<int2>(), C, lists.as<int>(), a->stride, nullptr, 1, sketch.as<signed char>(), nullptr, 1,
      scale.as<float>(), qs.as<float>(), S, W, logW, cand.as<int>(), dist.as<float>(), nin.as<int>());
    if (a->sketch_rank)  // search.cu:384
      ref::sketch_keep_kernel<<<m, 512>>>(cand.as<int>(), dist.as<float>(), nin.as<int>(), W, KO,
                                          si.as<long long>(), sd.as<float>(), true);
    else
      ref::rerank_keep_kernel<<<m, 256, D * sizeof(float)>>>(cand.as<int>(), dist.as<float>(), nin.as<int>(), W,
                                                             xptr.as<long long>(), a->n, D, q.as<float>(),
                                                             a->rerank, KO, si.as<long long>(), sd.as<float>(),
                                                             true);
    cudaEventRecord(ev[1]);
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    if (rep == reps - 1) {
      cudaMemcpy(a->seg, seg.p, sizeof(int2) * m * C, cudaMemcpyDeviceToHost);
      cudaMemcpy2D(a->cand1, sizeof(int) * a->w1, cand.p, sizeof(int) * W, sizeof(int) * W, m, cudaMemcpyDeviceToHost);
      cudaMemcpy2D(a->dist1, sizeof(float) * a->w1, dist.p, sizeof(float) * W, sizeof(float) * W, m,
                   cudaMemcpyDeviceToHost);
      cudaMemcpy(a->n1, nin.p, sizeof(int) * m, cudaMemcpyDeviceToHost);
      cudaMemcpy(a->kept1_ids, si.p, sizeof(long long) * m * KO, cudaMemcpyDeviceToHost);
      cudaMemcpy(a->kept1_dist, sd.p, sizeof(float) * m * KO, cudaMemcpyDeviceToHost);
    }
    float t = 0.f;
    cudaEventElapsedTime(&t, ev[0], ev[1]);
    ms1.push_back(t);

    // waves (search.cu:432-500): start points, their table rows, rerank into the kept list
    if (a->waves > 0) {
      flush_l2();
      cudaEventRecord(ev[2]);
      for (int wv = 0; wv < a->waves; wv++) {
        ref::pick_starts_kernel<<<m, 256>>>(si.as<long long>(), KO, done.as<long long>(), a->starts * a->waves,
                                            wv * a->starts, a->starts, a->table_len, seg2.as<int2>());
        ref::gather_kernel<true><<<m, 512, gather_smem(W2, S, a->starts)>>>(
          seg2.as<int2>(), a->starts, nullptr, a->table_len, tptr.as<long long>(), a->n, sketch.as<signed char>(),
          nullptr, 1, scale.as<float>(), qs.as<float>(), S, W2, logW2, cand2.as<int>(), dist2.as<float>(),
          n2.as<int>());
        if (a->sketch_rank)  // search.cu:479
          ref::sketch_keep_kernel<<<m, 512>>>(cand2.as<int>(), dist2.as<float>(), n2.as<int>(), W2, KO,
                                              si.as<long long>(), sd.as<float>(), false);
        else
          ref::rerank_keep_kernel<<<m, 256, D * sizeof(float)>>>(cand2.as<int>(), dist2.as<float>(), n2.as<int>(),
                                                                 W2, xptr.as<long long>(), a->n, D, q.as<float>(),
                                                                 a->wave_rerank, KO, si.as<long long>(),
                                                                 sd.as<float>(), false);
      }
      cudaEventRecord(ev[3]);
      e = cudaDeviceSynchronize();
      if (e != cudaSuccess) return static_cast<int>(e);
      cudaEventElapsedTime(&t, ev[2], ev[3]);
      ms2.push_back(t);
    }
  }
  if (a->kernel_ms != nullptr) {
    auto median = [](std::vector<float>& v) {
      if (v.empty()) return 0.f;
      std::sort(v.begin(), v.end());
      return v[v.size() / 2];
    };
    a->kernel_ms[0] = median(ms1);
    a->kernel_ms[1] = median(ms2);
  }
  for (auto& v : ev)
    cudaEventDestroy(v);
  cudaMemcpy(a->kept_ids, si.p, sizeof(long long) * m * KO, cudaMemcpyDeviceToHost);
  cudaMemcpy(a->kept_dist, sd.p, sizeof(float) * m * KO, cudaMemcpyDeviceToHost);
  // the result (search.cu:503-517)
  if (a->sketch_rank && FR > 0)
    ref::final_rerank_kernel<<<m, 256, D * sizeof(float)>>>(si.as<long long>(), KO, FR, xptr.as<long long>(), a->n,
                                                            D, q.as<float>(), a->k, bi.as<long long>(),
                                                            bd.as<float>());
  else
    ref::take_k_kernel<<<static_cast<unsigned>((int64_t{m} * a->k + 255) / 256), 256>>>(
      si.as<long long>(), sd.as<float>(), KO, a->k, m, bi.as<long long>(), bd.as<float>());
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaMemcpy(a->best_ids, bi.p, sizeof(long long) * m * a->k, cudaMemcpyDeviceToHost);
  cudaMemcpy(a->best_dist, bd.p, sizeof(float) * m * a->k, cudaMemcpyDeviceToHost);
  e = cudaGetLastError();
  return static_cast<int>(e);
}
