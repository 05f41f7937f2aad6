// TEST INFRASTRUCTURE ONLY. CPU restatement of the octex batched search path, used as the
// checker of the CUDA path and as the timed CPU baseline. The shipped library never links,
// loads or calls anything in this directory; it has no CPU fallback.
//
// Each step cites the reference code whose semantics it restates (paths inside hpdic/octex).
// Where the reference leaves an outcome open (the order of a candidate set, the choice among
// equal sketch distances at the rerank cut) this file picks the outcome "smallest
// (distance bits, id) first", which is one of the outcomes the reference allows.
//
// Parity pin: the E8 decode and cell code are checked against the reference's own e8.cuh
// compiled for the host and for the GPU (oracle/_ref, see the Makefile) and against the
// properties its unit test states (lattice membership, Voronoi optimality, hash_ref). The cell
// lookup, gather, sketch scoring, selection, exact rerank, kept-list merge and start-point choice
// are checked against the reference's own kernels (search_kernels.cuh compiled unmodified into
// oracle/_ref/libref_search.so and run on the GPU by tests/test_gpu_reference_kernels.py). The
// projection GEMM and the sketch-query GEMM run inside closed vendor libraries in the reference,
// so their rounding is not reproducible bit for bit: parity there is pinned by tolerance only.

#include "octex_oracle.h"

#include "e8_port.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <limits>
#include <queue>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_error;

using half_t = _Float16;

inline uint16_t half_bits(float v)
{
  half_t h = static_cast<half_t>(v);  // round to nearest even, as __float2half
  uint16_t b;
  std::memcpy(&b, &h, 2);
  return b;
}
inline float half_value(uint16_t b)
{
  half_t h;
  std::memcpy(&h, &b, 2);
  return static_cast<float>(h);
}
inline uint32_t float_bits(float v)
{
  uint32_t b;
  std::memcpy(&b, &v, 4);
  return b;
}
inline float bits_float(uint32_t b)
{
  float v;
  std::memcpy(&v, &b, 4);
  return v;
}

// (distance bits << 32) | low 32 bits of the id: the total order of every kept list
// (search_kernels.cuh:365-368).
inline uint64_t rank_key(float d, int64_t id)
{
  return (static_cast<uint64_t>(float_bits(d)) << 32) | static_cast<uint32_t>(id);
}
constexpr uint64_t kNoKey = ~0ULL;

template <typename F>
void parallel_rows(int64_t n, int threads, F&& body)
{
  int nt = threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency());
  nt     = std::max(1, std::min<int>(nt, static_cast<int>(std::max<int64_t>(n, 1))));
  if (nt == 1) {
    for (int64_t i = 0; i < n; i++)
      body(i, 0);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> pool;
  std::vector<std::string> errs(nt);
  for (int t = 0; t < nt; t++)
    pool.emplace_back([&, t] {
      try {
        for (;;) {
          int64_t i0 = next.fetch_add(16);
          if (i0 >= n) break;
          for (int64_t i = i0; i < std::min(n, i0 + 16); i++)
            body(i, t);
        }
      } catch (std::exception const& e) {
        errs[t] = e.what();
      }
    });
  for (auto& th : pool)
    th.join();
  for (auto& e : errs)
    if (!e.empty()) throw std::runtime_error(e);
}

// Operands of the projection as the loader prepares them (load.cu:385-402): projections and
// shifts rounded to fp16 (kept here as the floats those halves hold), 1 / spacing.
struct prepared {
  std::vector<float> u;      // [copies][dim][w]
  std::vector<float> shift;  // [copies][w]
  std::vector<float> inv_f;  // [levels]
};

prepared prepare(const oracle_index& ix)
{
  prepared p;
  const int w = 8 * ix.blocks;
  p.u.resize(static_cast<size_t>(ix.copies) * ix.dim * w);
  for (size_t i = 0; i < p.u.size(); i++)
    p.u[i] = half_value(half_bits(ix.proj[i]));
  p.shift.resize(static_cast<size_t>(ix.copies) * w);
  for (size_t i = 0; i < p.shift.size(); i++)
    p.shift[i] = half_value(half_bits(ix.shift[i]));
  for (int j = 0; j < ix.levels; j++)
    p.inv_f.push_back(static_cast<float>(1.0 / static_cast<double>(ix.spacings[j])));
  return p;
}

// Squared distance of an fp16 row to an fp32 query (search_kernels.cuh:325-342). Summation
// order shared with the CUDA path: element pair k feeds partial sum k mod 32 with two fused
// multiply-adds, then a butterfly over the 32 partial sums (strides 1, 2, 4, 8, 16).
float exact_distance(const uint16_t* row, const float* q, int dim)
{
  float part[32];
  for (int p = 0; p < 32; p++)
    part[p] = 0.f;
  const int pairs = dim / 2;
  for (int k = 0; k < pairs; k++) {
    float a = half_value(row[2 * k]) - q[2 * k];
    float b = half_value(row[2 * k + 1]) - q[2 * k + 1];
    float t = std::fma(a, a, part[k & 31]);
    part[k & 31] = std::fma(b, b, t);
  }
  for (int o = 1; o < 32; o <<= 1) {
    float nxt[32];
    for (int p = 0; p < 32; p++)
      nxt[p] = part[p] + part[p ^ o];
    std::memcpy(part, nxt, sizeof(part));
  }
  return part[0];
}

// int8 sketch distance sum_k (code_k * scale_k - qs_k)^2 (search_kernels.cuh:228-251):
// chunk c of 8 codes is partial sum c (two fused multiply-adds per code, in code order); a
// butterfly over Lr partial sums (strides 1, 2, 4, ...), Lr = the next power of two >= S / 8.
float sketch_distance(const int8_t* code, const float* scale, const float* qs, int S)
{
  int Lr = 1;
  while (Lr < S / 8)
    Lr <<= 1;  // S <= 512: at most 64 partial sums
  float part[64];
  for (int p = 0; p < Lr; p++)
    part[p] = 0.f;
  for (int c = 0; c * 8 < S; c++) {
    float d = 0.f;
    for (int t = 0; t < 8; t++) {
      int k   = c * 8 + t;
      float u = std::fma(static_cast<float>(code[k]), scale[k], -qs[k]);
      d       = std::fma(u, u, d);
    }
    part[c] = d;
  }
  for (int o = 1; o < Lr; o <<= 1) {
    float nxt[64];
    for (int p = 0; p < Lr; p++)
      nxt[p] = part[p] + part[p ^ o];
    std::memcpy(part, nxt, sizeof(float) * Lr);
  }
  return part[0];
}

// The same distance in the form the CUDA path evaluates it in the first round (where the candidates'
// rows are mostly cached and the arithmetic is what costs; in the waves it evaluates the sum above),
//   sum_k (c_k s_k - q_k)^2 = sum_k (c_k s_k)^2 - 2 sum_k c_k (s_k q_k) + sum_k q_k^2,
// with the middle sum in integers: per query the products t_k = s_k q_k are scaled to 16-bit
// weights w_k = rint(t_k / alpha), alpha = max |t_k| / 32000, so that sum_k c_k w_k is an exact
// int32 dot product of int8 codes with int16 weights; the first sum is a per-row constant and the
// last a per-query constant. Against the fp32 sum above the value differs by the rounding of the
// weights (relative 1.6e-5 of the largest product per term) and of three fp32 operations; every
// operation and its order are stated here and are the CUDA path's, so the two agree bit for bit.
struct sketch_query {
  std::vector<int32_t> w;  // [S] weights in [-32000, 32000]
  float beta = 0.f;        // -2 alpha
  float qq   = 0.f;        // sum of q_k^2: partial sum k mod 32, butterfly with strides 1 .. 16
};

sketch_query prepare_sketch_query(const float* scale, const float* qs, int S)
{
  sketch_query out;
  out.w.resize(S);
  std::vector<float> t(S);
  float amax = 0.f;
  for (int k = 0; k < S; k++) {
    t[k] = scale[k] * qs[k];
    amax = std::fmax(amax, std::fabs(t[k]));  // fmax ignores a NaN operand, as fmaxf on the GPU
  }
  const float alpha = (amax > 0.f && std::isfinite(amax)) ? amax / 32000.0f : 1.0f;
  for (int k = 0; k < S; k++) {
    const float r = std::nearbyint(t[k] / alpha);  // round to nearest even
    out.w[k] = std::isnan(r) ? 0 : static_cast<int32_t>(std::fmin(std::fmax(r, -32000.0f), 32000.0f));
  }
  out.beta = -2.0f * alpha;
  float part[32];
  for (int p = 0; p < 32; p++)
    part[p] = 0.f;
  for (int k = 0; k < S; k++)
    part[k & 31] = std::fma(qs[k], qs[k], part[k & 31]);
  for (int o = 1; o < 32; o <<= 1) {
    float nxt[32];
    for (int p = 0; p < 32; p++)
      nxt[p] = part[p] + part[p ^ o];
    std::memcpy(part, nxt, sizeof(part));
  }
  out.qq = part[0];
  return out;
}

// sum_k (c_k s_k)^2 of a row, one fused multiply-add per code in code order (a constant of the
// row: the CUDA path computes it when the index is placed).
float sketch_row_norm(const int8_t* code, const float* scale, int S)
{
  float n = 0.f;
  for (int k = 0; k < S; k++) {
    const float t = static_cast<float>(code[k]) * scale[k];
    n = std::fma(t, t, n);
  }
  return n;
}

float sketch_distance_int(const int8_t* code, float norm, const sketch_query& sq, int S)
{
  int32_t dot = 0;
  for (int k = 0; k < S; k++)
    dot += static_cast<int32_t>(code[k]) * sq.w[k];
  const float d = norm + std::fma(sq.beta, static_cast<float>(dot), sq.qq);
  return std::fmax(d, 0.f);  // rounding may leave a tiny negative value; keys order by bit pattern
}

struct kept_list {
  std::vector<int64_t> id;
  std::vector<float> d;
};

// Merge new (distance, id) pairs into a kept list of KO entries: ascending distinct keys, padded
// with (-1, +inf) (search_kernels.cuh:372-415).
void merge_kept(kept_list& kept, int KO, bool fresh, const std::vector<uint64_t>& fresh_keys)
{
  std::vector<uint64_t> keys;
  keys.reserve(KO + fresh_keys.size());
  if (!fresh)
    for (int i = 0; i < KO; i++)
      if (kept.id[i] >= 0) keys.push_back(rank_key(kept.d[i], kept.id[i]));
  keys.insert(keys.end(), fresh_keys.begin(), fresh_keys.end());
  std::sort(keys.begin(), keys.end());
  keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
  kept.id.assign(KO, -1);
  kept.d.assign(KO, std::numeric_limits<float>::infinity());
  for (int i = 0; i < KO && i < static_cast<int>(keys.size()); i++) {
    kept.id[i] = static_cast<int64_t>(static_cast<uint32_t>(keys[i] & 0xffffffffULL));
    kept.d[i]  = bits_float(static_cast<uint32_t>(keys[i] >> 32));
  }
}

// The R smallest of the candidates by (sketch distance bits, id) (search_kernels.cuh:259-322;
// the reference takes equal distances at the cut in any order).
std::vector<uint64_t> smallest(const std::vector<int32_t>& ids, const std::vector<float>& sd, int R)
{
  std::vector<uint64_t> keys(ids.size());
  for (size_t i = 0; i < ids.size(); i++)
    keys[i] = rank_key(sd[i], ids[i]);
  if (static_cast<int>(keys.size()) > R) {
    std::nth_element(keys.begin(), keys.begin() + R, keys.end());
    keys.resize(R);
  }
  std::sort(keys.begin(), keys.end());
  return keys;
}

struct scratch {
  std::vector<float> qc, y, qs;
  std::vector<uint16_t> qh, yh;
  std::vector<int32_t> ids;
  std::vector<float> sd;
};

}  // namespace

extern "C" {

const char* oracle_last_error(void) { return g_error.c_str(); }

int oracle_e8_point(const float* x, int64_t n_blocks, float* p)
{
  for (int64_t i = 0; i < n_blocks; i++)
    octex_oracle::nearest_e8(x + 8 * i, p + 8 * i);
  return 0;
}

int oracle_cell_code(const float* y, int64_t n, int32_t b, float inv_f, int64_t* h)
{
  for (int64_t i = 0; i < n; i++)
    h[i] = octex_oracle::cell_code(y + i * 8 * b, b, inv_f);
  return 0;
}

int oracle_to_half(const float* x, int64_t n, uint16_t* h)
{
  for (int64_t i = 0; i < n; i++)
    h[i] = half_bits(x[i]);
  return 0;
}

int oracle_from_half(const uint16_t* h, int64_t n, float* x)
{
  for (int64_t i = 0; i < n; i++)
    x[i] = half_value(h[i]);
  return 0;
}


int oracle_search(const oracle_index* ixp,
                  const oracle_params* spp,
                  const float* queries,
                  int64_t nq,
                  int32_t k,
                  int64_t* neighbors,
                  float* distances,
                  const oracle_taps* taps)
{
  try {
    const oracle_index& ix = *ixp;
    const oracle_params& sp = *spp;
    static const oracle_taps no_taps{};
    const oracle_taps& tp = taps ? *taps : no_taps;
    const int D = static_cast<int>(ix.dim), w = 8 * ix.blocks, C = ix.copies, L = ix.levels;
    const int S = ix.sketch_width, l = ix.list_len;
    const int64_t T1 = (int64_t{1} << ix.log_buckets) + 1;
    // limits and derived sizes: search.cu:625-655
    const int KO = std::max(sp.starts, k);
    const int lr = std::min(sp.read, l);
    const int FR = std::min(sp.final_rerank, KO);
    const int G  = std::max(1, sp.parts);
    if (k < 1) throw std::runtime_error("octex: k >= 1");
    if (sp.read < 1 || sp.starts < 1 || sp.waves < 0)
      throw std::runtime_error("octex: read, starts >= 1 and waves >= 0");
    if (sp.waves > 0 && ix.table_len <= 0)
      throw std::runtime_error("octex: waves need the neighbor table");
    if (G > C) throw std::runtime_error("octex: a device holds no copies");
    const prepared pre = prepare(ix);
    const int nthreads =
      sp.threads > 0 ? sp.threads : static_cast<int>(std::thread::hardware_concurrency());
    std::vector<scratch> work(std::max(1, nthreads));

    parallel_rows(nq, nthreads, [&](int64_t qi, int t) {
      scratch& sc    = work[t];
      const float* q = queries + qi * D;
      // centre, fp16 copy: search_kernels.cuh:57-69
      sc.qc.resize(D);
      sc.qh.resize(D);
      std::vector<float> qhf(D);
      for (int d = 0; d < D; d++) {
        sc.qc[d] = q[d] - ix.mean[d];
        sc.qh[d] = half_bits(sc.qc[d]);
        qhf[d]   = half_value(sc.qh[d]);
      }
      // projected coordinates Y = half(fp32(qh . u) + shift): search.cu:303-320
      sc.yh.resize(static_cast<size_t>(C) * w);
      if (tp.y_in) {
        std::memcpy(sc.yh.data(), tp.y_in + qi * C * w, sizeof(uint16_t) * C * w);
      } else {
        std::vector<float> acc(w);
        for (int c = 0; c < C; c++) {
          std::fill(acc.begin(), acc.end(), 0.f);
          const float* u = pre.u.data() + static_cast<size_t>(c) * D * w;
          for (int d = 0; d < D; d++) {
            const float a = qhf[d];
            const float* ur = u + static_cast<size_t>(d) * w;
            for (int s = 0; s < w; s++)
              acc[s] = std::fma(a, ur[s], acc[s]);
          }
          for (int s = 0; s < w; s++)
            sc.yh[c * w + s] = half_bits(acc[s] + pre.shift[c * w + s]);
        }
      }
      if (tp.y) std::memcpy(tp.y + qi * C * w, sc.yh.data(), sizeof(uint16_t) * C * w);
      // sketch-space query qs = qc @ basis: search.cu:321-341 (fp32 here, TF32 in the reference)
      sc.qs.assign(S, 0.f);
      for (int d = 0; d < D; d++) {
        const float a = sc.qc[d];
        const float* br = ix.basis + static_cast<size_t>(d) * S;
        for (int s = 0; s < S; s++)
          sc.qs[s] = std::fma(a, br[s], sc.qs[s]);
      }
      if (tp.qs) std::memcpy(tp.qs + qi * S, sc.qs.data(), sizeof(float) * S);

      int64_t st_levels = 0, st_keys = 0, st_entries = 0, st_n1 = 0, st_rows = 0, st_n2 = 0,
              st_exact = 0;
      // probe: the finest level whose cell holds a list (search_kernels.cuh:100-126)
      std::vector<int32_t> seg(2 * static_cast<size_t>(C), 0);
      std::vector<float> yf(w);
      for (int c = 0; c < C; c++) {
        for (int s = 0; s < w; s++)
          yf[s] = half_value(sc.yh[c * w + s]);
        bool found = false;
        for (int j = 0; j < L; j++) {
          int64_t h = octex_oracle::cell_code(yf.data(), ix.blocks, pre.inv_f[j]);
          if (tp.codes) tp.codes[(qi * C + c) * L + j] = h;
          if (found) continue;
          st_levels++;
          int64_t bk       = h & ((int64_t{1} << ix.log_buckets) - 1);
          const int32_t* o = ix.offsets + (static_cast<int64_t>(c) * L + j) * T1 + bk;
          const int64_t* kk = ix.keys + (static_cast<int64_t>(c) * L + j) * ix.mmax;
          for (int p = o[0]; p < o[1]; p++) {
            st_keys++;
            if (kk[p] == h) {
              seg[2 * c]     = (ix.base[c * L + j] + p) * l;
              seg[2 * c + 1] = lr;
              found          = true;
              break;
            }
          }
          if (found && !tp.codes) break;
        }
      }
      if (tp.seg) std::memcpy(tp.seg + qi * C * 2, seg.data(), sizeof(int32_t) * 2 * C);

      // The CUDA path scores the first round's candidates in the integer form and the waves' in
      // the fp32 sum when it reranks exactly; when it ranks by sketch distance (the distances of
      // all rounds meet in one kept list, where an id found twice must bring the same key both
      // times) every round takes the fp32 sum. sketch_form 1: the fp32 sum always, the reference's.
      const sketch_query sq = prepare_sketch_query(ix.scale, sc.qs.data(), S);
      auto score = [&](std::vector<int32_t>& ids, std::vector<float>& sd, bool first_round) {
        std::sort(ids.begin(), ids.end());
        ids.erase(std::unique(ids.begin(), ids.end()), ids.end());
        sd.resize(ids.size());
        for (size_t i = 0; i < ids.size(); i++) {
          const int8_t* row = ix.sketch + static_cast<int64_t>(ids[i]) * S;
          sd[i] = (sp.sketch_form == 1 || !first_round || sp.sketch_rank)
                    ? sketch_distance(row, ix.scale, sc.qs.data(), S)
                    : sketch_distance_int(row, sketch_row_norm(row, ix.scale, S), sq, S);
        }
      };
      auto keep = [&](kept_list& kept, bool fresh, int R) {
        // exact mode: rerank_keep_kernel (search_kernels.cuh:421-467);
        // sketch mode: sketch_keep_kernel (search_kernels.cuh:471-508)
        std::vector<uint64_t> sel = smallest(sc.ids, sc.sd, sp.sketch_rank ? KO : R);
        if (!sp.sketch_rank) {
          for (auto& key : sel) {
            int32_t id = static_cast<int32_t>(key & 0xffffffffULL);
            float d    = exact_distance(ix.vectors + static_cast<int64_t>(id) * D, q, D);
            key        = rank_key(d, id);
            st_exact++;
          }
        }
        merge_kept(kept, KO, fresh, sel);
      };

      // first round per part (search.cu:294-407); parts > 1 emulate the sharded placement
      std::vector<kept_list> part_kept(G);
      int cand_at = 0;
      for (int g = 0; g < G; g++) {
        const int c0 = static_cast<int>(int64_t{C} * g / G), c1 = static_cast<int>(int64_t{C} * (g + 1) / G);
        sc.ids.clear();
        for (int c = c0; c < c1; c++) {
          const int32_t* lp = ix.lists + static_cast<int64_t>(c) * ix.stride + seg[2 * c];
          for (int i = 0; i < seg[2 * c + 1]; i++)
            sc.ids.push_back(lp[i]);
          st_entries += seg[2 * c + 1];
        }
        score(sc.ids, sc.sd, true);
        st_n1 += static_cast<int64_t>(sc.ids.size());
        if (tp.cand1) {
          for (size_t i = 0; i < sc.ids.size() && cand_at < tp.cand_cap; i++, cand_at++) {
            tp.cand1[qi * tp.cand_cap + cand_at] = sc.ids[i];
            if (tp.cand1_dist) tp.cand1_dist[qi * tp.cand_cap + cand_at] = sc.sd[i];
          }
        }
        part_kept[g].id.assign(KO, -1);
        part_kept[g].d.assign(KO, std::numeric_limits<float>::infinity());
        keep(part_kept[g], true, sp.rerank);
      }
      if (tp.n1) tp.n1[qi] = cand_at;
      kept_list kept;
      if (G == 1) {
        kept = std::move(part_kept[0]);
      } else {
        // merge_kept_kernel (search_kernels.cuh:517-564): the nearest copy of each id, best KO
        std::vector<uint64_t> by_id;
        for (auto& pk : part_kept)
          for (int i = 0; i < KO; i++)
            if (pk.id[i] >= 0)
              by_id.push_back((static_cast<uint64_t>(static_cast<uint32_t>(pk.id[i])) << 32) |
                              float_bits(pk.d[i]));
        std::sort(by_id.begin(), by_id.end());
        std::vector<uint64_t> keys;
        for (size_t i = 0; i < by_id.size(); i++)
          if (i == 0 || (by_id[i - 1] >> 32) != (by_id[i] >> 32))
            keys.push_back(((by_id[i] & 0xffffffffULL) << 32) | (by_id[i] >> 32));
        kept.id.assign(KO, -1);
        kept.d.assign(KO, std::numeric_limits<float>::infinity());
        merge_kept(kept, KO, true, keys);
      }
      if (tp.kept1_ids) std::memcpy(tp.kept1_ids + qi * KO, kept.id.data(), sizeof(int64_t) * KO);
      if (tp.kept1_dist) std::memcpy(tp.kept1_dist + qi * KO, kept.d.data(), sizeof(float) * KO);

      // waves (search.cu:451-502): start points not expanded before (search_kernels.cuh:571-631),
      // their table rows, rerank, merge
      std::vector<int64_t> done;
      for (int wv = 0; wv < sp.waves; wv++) {
        std::vector<int64_t> starts;
        for (int i = 0; i < KO && static_cast<int>(starts.size()) < sp.starts; i++) {
          int64_t v = kept.id[i];
          if (v < 0) continue;
          if (std::find(done.begin(), done.end(), v) != done.end()) continue;
          starts.push_back(v);
        }
        done.insert(done.end(), starts.begin(), starts.end());
        sc.ids.clear();
        for (int64_t row : starts) {
          const int32_t* tr = ix.table + row * ix.table_len;
          for (int i = 0; i < ix.table_len; i++)
            if (tr[i] >= 0) sc.ids.push_back(tr[i]);
        }
        st_rows += static_cast<int64_t>(starts.size());
        score(sc.ids, sc.sd, false);
        st_n2 += static_cast<int64_t>(sc.ids.size());
        keep(kept, false, sp.wave_rerank);
      }
      // best k: final_rerank_kernel / take_k_kernel (search_kernels.cuh:634-685)
      if (sp.sketch_rank && FR > 0) {
        std::vector<uint64_t> keys;
        for (int i = 0; i < FR; i++)
          if (kept.id[i] >= 0) {
            float d = exact_distance(ix.vectors + kept.id[i] * D, q, D);
            keys.push_back(rank_key(d, kept.id[i]));
            st_exact++;
          }
        kept_list out;
        out.id.assign(k, -1);
        out.d.assign(k, std::numeric_limits<float>::infinity());
        merge_kept(out, k, true, keys);
        std::memcpy(neighbors + qi * k, out.id.data(), sizeof(int64_t) * k);
        std::memcpy(distances + qi * k, out.d.data(), sizeof(float) * k);
      } else {
        std::memcpy(neighbors + qi * k, kept.id.data(), sizeof(int64_t) * k);
        std::memcpy(distances + qi * k, kept.d.data(), sizeof(float) * k);
      }
      if (tp.stats) {
        int64_t* s = tp.stats + qi * 8;
        s[0] = st_levels; s[1] = st_keys; s[2] = st_entries; s[3] = st_n1;
        s[4] = st_rows; s[5] = st_n2; s[6] = st_exact; s[7] = 0;
      }
    });
    g_error.clear();
    return 0;
  } catch (std::exception const& e) {
    g_error = e.what();
    return 1;
  }
}

int oracle_brute_force(const float* base, int64_t n, int64_t dim, const float* queries, int64_t nq,
                       int32_t k, int32_t threads, int64_t* ids, float* dist)
{
  try {
    parallel_rows(nq, threads, [&](int64_t qi, int) {
      const float* q = queries + qi * dim;
      std::priority_queue<std::pair<double, int64_t>> heap;  // largest on top
      for (int64_t i = 0; i < n; i++) {
        const float* x = base + i * dim;
        double d = 0;
        for (int64_t t = 0; t < dim; t++) {
          double e = static_cast<double>(x[t]) - static_cast<double>(q[t]);
          d += e * e;
        }
        if (static_cast<int>(heap.size()) < k) {
          heap.emplace(d, i);
        } else if (std::make_pair(d, i) < heap.top()) {
          heap.pop();
          heap.emplace(d, i);
        }
      }
      for (int j = static_cast<int>(heap.size()); j < k; j++) {
        ids[qi * k + j]  = -1;
        dist[qi * k + j] = std::numeric_limits<float>::infinity();
      }
      for (int j = static_cast<int>(heap.size()) - 1; j >= 0; j--) {
        ids[qi * k + j]  = heap.top().second;
        dist[qi * k + j] = static_cast<float>(heap.top().first);
        heap.pop();
      }
    });
    g_error.clear();
    return 0;
  } catch (std::exception const& e) {
    g_error = e.what();
    return 1;
  }
}

}  // extern "C"
