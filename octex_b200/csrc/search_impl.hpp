// Buffers and graph of one batch shape and one set of search parameters (the reference's
// plan / gpu_plan, cpp/src/neighbors/octex/search.cu:35-80 of hpdic/octex, for one GPU).
#pragma once

#include "index_impl.hpp"
#include "kernels.hpp"

#include <mutex>
#include <vector>

namespace octex_b200::detail {

struct plan {
  search_params sp;
  debug_options dbg;
  int device = 0;
  int m = 0, k = 0, KO = 0, lr = 0, R1 = 0, R2 = 0, FR = 0;
  // Who answers what in a batch of m rows when `world` processes share the index
  // (search.cu:666-676 of the reference, per GPU there, per process here): the first round runs on
  // rows [q1, q1 + m1) — all m rows when the copies are sharded, the own slice otherwise — and the
  // waves on the own slice [lo, hi).
  int rank = 0, world = 1;
  bool shard = false;
  int m1 = 0, q1 = 0, lo = 0, hi = 0, mw = 0, mwmax = 0;
  dbuf si2, sd2;        // shard: kept list of the own slice after the cross-process merge
  dbuf recv_i, recv_d;  // shard: [world, mwmax, KO] first-round kept lists of every process
  dbuf out;             // results of this process's slice: ids [mwmax, k], then distances [mwmax, k]
  dbuf gathered;        // world > 1: the out blocks of every process
  size_t out_block = 0, out_ids = 0;  // bytes of a block and of its ids
  long long* bi = nullptr;            // the two arrays inside out
  float* bd     = nullptr;
  long long* wsi = nullptr;  // kept list the waves work on [mw, KO]
  float* wsd     = nullptr;
  int P_merge    = 0;   // keys sorted by the cross-process merge (power of two >= world * KO)
  dbuf qbuf, qh, qs, Y, codes, seg, si, sd, done, stats, phase1, phase2;
  dbuf tap_cand, tap_dist, tap_n, kept1_i, kept1_d;
  bool use_tc = false;          // tensor-core projection with the decode in its epilogue
  kernels::project_tc_plan tc;  // its tensor maps
  int* tc_error_host = nullptr; // pinned, device-visible: non-zero when a bounded wait in a kernel ran out
  int* tc_error_dev  = nullptr;
  int tap_cap = 0;
  std::vector<dbuf> scratch_cand, scratch_dist;
  kernels::round_args r1, r2;
  size_t smem_max       = 0;
  cudaGraphExec_t graph = nullptr;
  cudaEvent_t done_ev   = nullptr;
  cudaEvent_t start_ev  = nullptr;  // recorded on the caller's stream at the start of a search
  int start_dev         = -1;       // device it was created on
  int64_t buffer_bytes  = 0;
  std::mutex mu;  // one search at a time per plan
  ~plan();
};

inline auto ix_debug(index_impl const& ix) -> debug_options { return ix.debug; }

void search_impl(resources const& res,
                 search_params const& sp,
                 index const& idx,
                 const float* queries,
                 int64_t nq,
                 int64_t qdim,
                 int64_t* neighbors,
                 float* distances,
                 int64_t k,
                 bool host_out,
                 bool resident);

/// One batch of the queries already on the GPU, launched kernel by kernel with an event between
/// them: milliseconds of center+sketch, projection, cell codes, lookup, first round, each wave,
/// best k (the per-kernel counterpart of detail::timed_batch, search.cu:965-981 of the reference).
auto profile_batch(resources const& res, search_params const& sp, index const& idx, int64_t nq,
                   int64_t k) -> std::vector<float>;

/// Throws when a kernel of an earlier batch of this plan reported that it gave up (and clears the
/// report).
void check_tc(plan const& pl);

auto get_plan(index_impl& ix, search_params const& sp, int m, int k, int lane = 0) -> std::shared_ptr<plan>;

}  // namespace octex_b200::detail
