// Batched search: plan (limits, buffers, one CUDA graph per batch shape) and the per-batch loop.
//
// Answers cpp/src/neighbors/octex/search.cu of hpdic/octex (make_plan :619-794, get_plan :796-814,
// search_impl :816-961, the two search overloads :1020-1064) for one process per GPU. Parameter
// limits and error texts are the reference's. A batch is: copy the queries in, pad a partial batch
// with copies of its first row, replay the graph (centre + sketch-space query, projection, cell
// codes, cell lookup, first round, waves, best k), copy the results out.

#include "search_impl.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace octex_b200 {

namespace detail {

namespace {

template <typename T>
auto alloc(plan& pl, int device, int64_t count, int fill = -2) -> dbuf
{
  dbuf b(device, static_cast<size_t>(std::max<int64_t>(count, 1)) * sizeof(T));
  if (fill != -2) OCTEX_CUDA_TRY(cudaMemset(b.ptr, fill, b.size));
  pl.buffer_bytes += static_cast<int64_t>(b.size);
  return b;
}

/// The kernels' view of an array dealt by rows (empty when the array is whole).
auto map_of(index_impl const& ix, dealt_rows const& d) -> kernels::row_map
{
  kernels::row_map m;
  if (!d.on) return m;
  OCTEX_EXPECTS(d.ptrs.ptr != nullptr,
                "octex: the index holds row ranges of other processes: connect the processes first "
                "(octexB200CommInit)");
  OCTEX_EXPECTS(d.rows_per < (int64_t{1} << 31), "octex: more than 2^31 rows per process");
  m.ptrs  = d.ptrs.as<long long>();
  m.rows  = static_cast<int>(d.rows_per);
  m.local = static_cast<int>(std::min<int64_t>(d.row0, ix.n - 1));
  return m;
}

constexpr size_t kSmemSoftLimit = size_t{96} << 10;   // above this the candidates go to global memory
constexpr size_t kSmemHardLimit = size_t{227} << 10;  // shared memory a block can opt in to

/// Fill the size fields of a round and decide where its candidate arrays live.
void size_round(plan& pl, kernels::round_args& r, int entries_max, int pick_entries, int device,
                int64_t sketch_bytes)
{
  r.pick_slots = 0;
  if (pick_entries > 0) {
    r.pick_slots = 64;
    while (r.pick_slots * 3 < pick_entries * 4)  // at most 75 % full
      r.pick_slots <<= 1;
  }
  int kept_slots = 64;  // the set of kept ids a round filters its selection with
  while (kept_slots < 2 * r.KO)
    kept_slots <<= 1;
  r.nmax = std::max(entries_max, 1);
  r.P    = 2;
  while (r.P < r.KO)
    r.P <<= 1;
  r.cand_global = nullptr;
  r.dist_global = nullptr;
  // the gather's hash set: half full at most when eight blocks still fit a multiprocessor's shared
  // memory (1 KB per block is the system's), else two thirds, else three quarters
  constexpr size_t kEightBlocks = (size_t{228} << 10) / 8 - 1024;
  for (int twelfths : {24, 18, 16}) {
    r.hash_twelfths = twelfths;
    r.cap_slots = kernels::hash_slots_of(std::min(entries_max, kernels::kMaxHash), kernels::kMaxHash, twelfths);
    r.ht_slots  = std::max({r.cap_slots, r.pick_slots, kept_slots});
    if (kernels::round_smem_bytes(r) <= kEightBlocks) break;
  }
  if (kernels::round_smem_bytes(r) > kSmemSoftLimit) {
    // placeholders: non-null makes the layout drop the two arrays; the real buffers follow
    r.cand_global = reinterpret_cast<int*>(1);
    r.dist_global = reinterpret_cast<float*>(1);
    OCTEX_EXPECTS(kernels::round_smem_bytes(r) <= kSmemHardLimit,
                  "octex: the round does not fit shared memory");
    pl.scratch_cand.push_back(alloc<int>(pl, device, int64_t{r.m} * r.nmax));
    r.cand_global = pl.scratch_cand.back().as<int>();
    // the sketch distances still go where the hash set was when that region holds them all (the
    // selection makes several passes over them)
    r.dist_global = nullptr;
    if (r.ht_slots < r.nmax) {
      pl.scratch_dist.push_back(alloc<float>(pl, device, int64_t{r.m} * r.nmax));
      r.dist_global = pl.scratch_dist.back().as<float>();
    }
  }
  pl.smem_max = std::max(pl.smem_max, kernels::round_smem_bytes(r));
  // threads per block: a multiprocessor runs 1024 threads of this kernel (64 registers each); when
  // fewer than eight blocks fit its shared memory, the blocks get more threads to make up for it
  const size_t per_block = kernels::round_smem_bytes(r) + 1024;
  const int fit          = static_cast<int>(std::max<size_t>((size_t{228} << 10) / per_block, 1));
  r.threads              = fit >= 8 ? 128 : fit >= 4 ? 256 : 512;
  {
    // the sketch stays in the L2 cache when it and its constants take at most 60 % of it
    int l2 = 0;
    OCTEX_CUDA_TRY(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, device));
    r.keep_sketch = sketch_bytes > 0 && static_cast<double>(sketch_bytes) <= 0.6 * l2 ? 1 : 0;
  }
}

}  // namespace

plan::~plan()
{
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(device);
  if (graph != nullptr) cudaGraphExecDestroy(graph);
  if (done_ev != nullptr) cudaEventDestroy(done_ev);
  if (start_ev != nullptr) cudaEventDestroy(start_ev);
  if (tc_error_host != nullptr) cudaFreeHost(tc_error_host);
  cudaSetDevice(cur);
}

/// A wait inside the tensor-core projection gave up (it never does unless the GPU misbehaves):
/// report it once and clear the word, so that one event does not poison the calls after it. Call
/// it when the stream of the plan is idle.
void check_tc(plan const& pl)
{
  if (pl.tc_error_host == nullptr || *pl.tc_error_host == 0) return;
  const int code    = *pl.tc_error_host;
  *pl.tc_error_host = 0;
  throw error("octex: a kernel gave up waiting for data it had asked for (code " + std::to_string(code) +
              ": 1, 2 the projection's operands, 3 the segments of a gather, 4 the rows of a rerank); "
              "the results of that batch are not valid");
}

/// Launch every kernel of a batch on s (captured into the graph, or run directly).
void run_batch(index_impl const& ix, plan& pl, cudaStream_t s, std::vector<cudaEvent_t>* marks)
{
  // marks (profiling only): one event before the first kernel and one after every kernel
  auto mark = [&] {
    if (marks == nullptr) return;
    cudaEvent_t e = nullptr;
    OCTEX_CUDA_TRY(cudaEventCreate(&e));
    OCTEX_CUDA_TRY(cudaEventRecord(e, s));
    marks->push_back(e);
  };
  auto const& p  = ix.part;
  const int D    = static_cast<int>(ix.dim);
  const int sw   = ix.sketch_width;
  const int L    = static_cast<int>(ix.spacings.size());
  const int wdt  = 8 * ix.blocks * p.copies;
  if (pl.stats.ptr != nullptr) {
    OCTEX_CUDA_TRY(cudaMemsetAsync(pl.stats.ptr, 0, pl.stats.size, s));
    OCTEX_CUDA_TRY(cudaMemsetAsync(pl.phase1.ptr, 0, pl.phase1.size, s));
    OCTEX_CUDA_TRY(cudaMemsetAsync(pl.phase2.ptr, 0, pl.phase2.size, s));
  }
  mark();
  kernels::center_sketch(pl.qbuf.as<float>(), p.mean.as<float>(), p.basis.as<float>(), pl.m1, D, sw,
                         pl.qh.as<__half>(), p.ldu, pl.qs.as<float>(), s);
  mark();
  const unsigned char* levels = pl.dbg.taps ? nullptr : p.level_on.as<unsigned char>();
  // without inspection the cells are looked up where their codes are computed: no codes array, no
  // lookup kernel
  const bool fused_lookup = pl.use_tc && !pl.dbg.taps;
  if (pl.use_tc) {
    // tensor cores; the projected coordinates stay in TMEM unless they are asked for
    float finest = ix.spacings[0];
    for (float f : ix.spacings)
      finest = std::min(finest, f);
    kernels::tc_lookup look;
    if (fused_lookup) {
      look.table    = p.cell_table.as<kernels::cell_slot>();
      look.toff     = p.cell_off.as<long long>();
      look.tmask    = p.cell_mask.as<int>();
      look.base     = p.base.as<int>();
      look.list_len = ix.list_len;
      look.lr       = pl.lr;
      look.seg      = pl.seg.as<int2>();
      look.stats    = pl.stats.as<long long>();
    }
    kernels::project_decode_tc(pl.tc, L, p.shift.as<__half>(), p.inv_f.as<float>(), finest, levels,
                               pl.codes.as<long long>(), pl.dbg.taps ? pl.Y.as<__half>() : nullptr, look,
                               pl.tc_error_dev, s);
    mark();
  } else {
    kernels::project_ordered(pl.qh.as<__half>(), p.ldu, p.ut.as<__half>(), p.ldu,
                             p.shift.as<__half>(), pl.m1, wdt, D, pl.Y.as<__half>(), s);
    mark();
    kernels::decode_codes(pl.Y.as<__half>(), int64_t{pl.m1} * p.copies, p.copies, ix.blocks, L,
                          p.inv_f.as<float>(), levels, pl.codes.as<long long>(), s);
  }
  mark();
  if (!fused_lookup)
    kernels::probe(pl.codes.as<long long>(), pl.m1, p.copies, L, p.cell_table.as<kernels::cell_slot>(),
                   p.cell_off.as<long long>(), p.cell_mask.as<int>(), p.base.as<int>(),
                   p.level_on.as<unsigned char>(), ix.list_len, pl.lr, pl.seg.as<int2>(),
                   pl.stats.as<long long>(), s);
  mark();
  kernels::round_lists(pl.r1, s);
  mark();
  if (pl.shard) {
    // Every process ran the first round of all m rows over its own copies. Row block [lo_r, hi_r)
    // of each kept list goes to process r (search_kernels.cuh:517-539 reads the same blocks through
    // peer pointers); then the nearest copy of every id, best KO (merge_kept_kernel).
    auto& c        = *ix.comm;
    const size_t e = static_cast<size_t>(pl.KO);
    c.group_start();
    for (int r = 0; r < pl.world; r++) {
      const int lo_r = static_cast<int>(int64_t{pl.m} * r / pl.world);
      const int hi_r = static_cast<int>(int64_t{pl.m} * (r + 1) / pl.world);
      long long* ri  = pl.recv_i.as<long long>() + static_cast<size_t>(r) * pl.mwmax * e;
      float* rd      = pl.recv_d.as<float>() + static_cast<size_t>(r) * pl.mwmax * e;
      if (r == pl.rank) {
        OCTEX_CUDA_TRY(cudaMemcpyAsync(ri, pl.si.as<long long>() + pl.lo * e, pl.mw * e * sizeof(long long),
                                       cudaMemcpyDeviceToDevice, s));
        OCTEX_CUDA_TRY(cudaMemcpyAsync(rd, pl.sd.as<float>() + pl.lo * e, pl.mw * e * sizeof(float),
                                       cudaMemcpyDeviceToDevice, s));
        continue;
      }
      c.send(pl.si.as<long long>() + lo_r * e, (hi_r - lo_r) * e * sizeof(long long), r, s);
      c.send(pl.sd.as<float>() + lo_r * e, (hi_r - lo_r) * e * sizeof(float), r, s);
      c.recv(ri, pl.mw * e * sizeof(long long), r, s);
      c.recv(rd, pl.mw * e * sizeof(float), r, s);
    }
    c.group_end();
    mark();
    kernels::merge_kept(pl.recv_i.as<long long>(), pl.recv_d.as<float>(), pl.world,
                        int64_t{pl.mwmax} * pl.KO, pl.KO, pl.P_merge, pl.mw, pl.wsi, pl.wsd, s);
    mark();
  }
  if (pl.dbg.taps && pl.mw > 0) {
    OCTEX_CUDA_TRY(cudaMemcpyAsync(pl.kept1_i.ptr, pl.wsi, sizeof(long long) * pl.mw * pl.KO,
                                   cudaMemcpyDeviceToDevice, s));
    OCTEX_CUDA_TRY(cudaMemcpyAsync(pl.kept1_d.ptr, pl.wsd, sizeof(float) * pl.mw * pl.KO,
                                   cudaMemcpyDeviceToDevice, s));
  }
  const float* Qw = pl.qbuf.as<float>() + static_cast<size_t>(pl.lo - pl.q1) * D;
  for (int wv = 0; wv < pl.sp.waves; wv++) {
    kernels::round_args r = pl.r2;
    r.done_off            = wv * pl.sp.starts;
    kernels::round_rows(r, s);
    mark();
  }
  if (pl.sp.sketch_rank && pl.FR > 0) {
    kernels::final_rerank(pl.wsi, pl.KO, pl.FR, p.vectors.as<__half>(), pl.r1.vector_map, D, Qw, pl.k,
                          pl.mw, pl.bi, pl.bd, pl.stats.as<long long>(), s);
  } else {
    kernels::take_k(pl.wsi, pl.wsd, pl.KO, pl.k, pl.mw, pl.bi, pl.bd, s);
  }
  mark();
  if (pl.world > 1) {
    // every process gets the results of all slices (blocks of mwmax rows, the last rows of a
    // block unused when the slices differ in size)
    ix.comm->all_gather(pl.out.ptr, pl.gathered.ptr, pl.out_block, s);
    mark();
  }
  OCTEX_CUDA_TRY(cudaPeekAtLastError());
}

auto profile_batch(resources const& res, search_params const& sp, index const& idx, int64_t nq,
                   int64_t k) -> std::vector<float>
{
  auto& ix = idx.impl();
  OCTEX_EXPECTS(nq >= 1 && nq <= std::max(sp.batch, 1),
                "octex: a profiled batch is one batch of queries already on the GPU");
  (void)res;
  auto pl = get_plan(ix, sp, static_cast<int>(nq), static_cast<int>(k));
  std::lock_guard<std::mutex> lock(pl->mu);
  int cur = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  OCTEX_CUDA_TRY(cudaSetDevice(ix.part.device));
  std::vector<cudaEvent_t> marks;
  std::vector<float> ms;
  try {
    run_batch(ix, *pl, ix.part.stream, &marks);
    OCTEX_CUDA_TRY(cudaStreamSynchronize(ix.part.stream));
    for (size_t i = 1; i < marks.size(); i++) {
      float t = 0.f;
      OCTEX_CUDA_TRY(cudaEventElapsedTime(&t, marks[i - 1], marks[i]));
      ms.push_back(t);
    }
  } catch (...) {
    for (auto e : marks)
      cudaEventDestroy(e);
    cudaSetDevice(cur);
    throw;
  }
  for (auto e : marks)
    cudaEventDestroy(e);
  OCTEX_CUDA_TRY(cudaSetDevice(cur));
  return ms;
}

auto make_plan(index_impl& ix, search_params const& sp, int m, int k, debug_options dbg)
  -> std::shared_ptr<plan>
{
  auto plp  = std::make_shared<plan>();
  plan& pl  = *plp;
  auto& p   = ix.part;
  pl.sp     = sp;
  pl.dbg    = dbg;
  pl.m      = m;
  pl.k      = k;
  pl.KO     = std::max(sp.starts, k);
  pl.lr     = std::min(sp.read, ix.list_len);
  pl.R1     = sp.rerank;
  pl.R2     = sp.wave_rerank;
  pl.FR     = std::min(sp.final_rerank, pl.KO);
  pl.device = p.device;
  const int D  = static_cast<int>(ix.dim);
  const int sw = ix.sketch_width;
  const int S  = sp.starts;
  const int L  = static_cast<int>(ix.spacings.size());
  // search.cu:637-655
  OCTEX_EXPECTS(sp.read >= 1 && sp.starts >= 1 && sp.waves >= 0,
                "octex: read, starts >= 1 and waves >= 0");
  OCTEX_EXPECTS(sp.waves == 0 || ix.table_len > 0, "octex: waves need the neighbor table");
  OCTEX_EXPECTS(pl.KO <= (sp.sketch_rank ? kernels::kMaxSketchKO : kernels::kMaxRerank),
                "octex: max(starts, k) must be <= 512 (1024 with sketch_rank)");
  OCTEX_EXPECTS(sp.sketch_rank || (sp.rerank >= 1 && sp.rerank <= kernels::kMaxRerank &&
                                   pl.KO + sp.rerank <= kernels::kMaxKeepSort),
                "octex: rerank in [1, 512] and max(starts, k) + rerank <= 1024");
  OCTEX_EXPECTS(sp.sketch_rank || sp.waves == 0 ||
                  (sp.wave_rerank >= 1 && sp.wave_rerank <= kernels::kMaxRerank &&
                   pl.KO + sp.wave_rerank <= kernels::kMaxKeepSort),
                "octex: wave_rerank in [1, 512] and max(starts, k) + wave_rerank <= 1024");
  OCTEX_EXPECTS(!sp.sketch_rank || pl.FR == 0 || (k <= pl.FR && pl.FR <= kernels::kMaxRerank),
                "octex: final_rerank 0 (sketch order) or k <= final_rerank <= 512");
  OCTEX_EXPECTS(sp.waves <= 1 || S * (sp.waves - 1) <= kernels::kMaxExpanded,
                "octex: starts * (waves - 1) <= 6144");
  OCTEX_EXPECTS(int64_t{p.copies} * pl.lr <= kernels::kMaxHash,
                "octex: copies x read too large for the shared-memory hash set");
  OCTEX_EXPECTS(sp.waves == 0 || int64_t{S} * ix.table_len <= kernels::kMaxHash,
                "octex: starts x table_len too large for the shared-memory hash set");
  // slices (search.cu:666-676 of the reference)
  pl.rank  = ix.rank;
  pl.world = ix.world;
  pl.shard = ix.params.mode == placement::shard && ix.world > 1;
  OCTEX_EXPECTS(ix.world == 1 || ix.comm != nullptr,
                "octex: an index shared by several processes needs its communicator first "
                "(octexB200CommInit)");
  OCTEX_EXPECTS(!pl.shard || ix.world * pl.KO <= 4096, "octex: devices * max(starts, k) <= 4096");
  pl.lo    = static_cast<int>(int64_t{m} * ix.rank / ix.world);
  pl.hi    = static_cast<int>(int64_t{m} * (ix.rank + 1) / ix.world);
  pl.mw    = pl.hi - pl.lo;
  pl.mwmax = (m + ix.world - 1) / ix.world;
  pl.q1    = pl.shard ? 0 : pl.lo;
  pl.m1    = pl.shard ? m : pl.mw;

  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  const int m1  = std::max(pl.m1, 1);
  const int wdt = 8 * ix.blocks * p.copies;
  pl.qbuf  = alloc<float>(pl, p.device, int64_t{m1} * D, 0);
  pl.qh    = alloc<__half>(pl, p.device, int64_t{m1} * p.ldu);
  pl.qs    = alloc<float>(pl, p.device, int64_t{m1} * sw);
  pl.use_tc = !dbg.ordered_projection && kernels::project_tc_supported(ix.blocks, p.ldu);
  if (!pl.use_tc || dbg.taps) pl.Y = alloc<__half>(pl, p.device, int64_t{m1} * wdt);
  // the word a kernel sets when one of its bounded waits (on an mbarrier) ran out
  OCTEX_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&pl.tc_error_host), sizeof(int), cudaHostAllocMapped));
  *pl.tc_error_host = 0;
  OCTEX_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&pl.tc_error_dev), pl.tc_error_host, 0));
  if (pl.use_tc) {
    kernels::project_tc_setup(pl.tc, pl.qh.as<__half>(), m1, p.ut.as<__half>(), p.copies, p.ldu);
  }
  pl.codes = alloc<long long>(pl, p.device, int64_t{m1} * p.copies * L);
  pl.seg   = alloc<int2>(pl, p.device, int64_t{m1} * p.copies);
  pl.si    = alloc<long long>(pl, p.device, int64_t{m1} * pl.KO, 0xff);
  pl.sd    = alloc<float>(pl, p.device, int64_t{m1} * pl.KO);
  const int mwmax = std::max(pl.mwmax, 1);
  // the results of this process's slice: ids [mwmax, k], then distances [mwmax, k], in one block so
  // that one collective moves both
  pl.out_ids = sizeof(long long) * static_cast<size_t>(mwmax) * k;
  pl.out_block = pl.out_ids + sizeof(float) * static_cast<size_t>(mwmax) * k;
  pl.out   = alloc<char>(pl, p.device, static_cast<int64_t>(pl.out_block), 0xff);
  pl.bi    = pl.out.as<long long>();
  pl.bd    = reinterpret_cast<float*>(pl.out.as<char>() + pl.out_ids);
  pl.wsi   = pl.si.as<long long>();
  pl.wsd   = pl.sd.as<float>();
  if (pl.shard) {
    pl.si2    = alloc<long long>(pl, p.device, int64_t{mwmax} * pl.KO, 0xff);
    pl.sd2    = alloc<float>(pl, p.device, int64_t{mwmax} * pl.KO);
    pl.recv_i = alloc<long long>(pl, p.device, int64_t{ix.world} * mwmax * pl.KO, 0xff);
    pl.recv_d = alloc<float>(pl, p.device, int64_t{ix.world} * mwmax * pl.KO, 0);
    pl.wsi    = pl.si2.as<long long>();
    pl.wsd    = pl.sd2.as<float>();
    pl.P_merge = 2;
    while (pl.P_merge < ix.world * pl.KO)
      pl.P_merge <<= 1;
  }
  if (ix.world > 1) {
    pl.gathered = alloc<char>(pl, p.device, static_cast<int64_t>(pl.out_block) * ix.world, 0xff);
  }
  if (sp.waves > 0) pl.done = alloc<int>(pl, p.device, int64_t{m1} * S * sp.waves, 0xff);
  if (dbg.stats) {
    pl.stats  = alloc<long long>(pl, p.device, int64_t{m1} * 8, 0);
    pl.phase1 = alloc<long long>(pl, p.device, int64_t{m1} * 8, 0);
    pl.phase2 = alloc<long long>(pl, p.device, int64_t{m1} * 8, 0);
  }
  if (dbg.taps) {
    pl.tap_cap  = p.copies * pl.lr;
    pl.tap_cand = alloc<int>(pl, p.device, int64_t{m1} * pl.tap_cap, 0xff);
    pl.tap_dist = alloc<float>(pl, p.device, int64_t{m1} * pl.tap_cap, 0);
    pl.tap_n    = alloc<int>(pl, p.device, m1, 0);
    pl.kept1_i  = alloc<long long>(pl, p.device, int64_t{m1} * pl.KO, 0xff);
    pl.kept1_d  = alloc<float>(pl, p.device, int64_t{m1} * pl.KO, 0);
  }

  // first round: lists of this process's copies
  auto& r1       = pl.r1;
  r1.m           = pl.m1;
  r1.nseg        = p.copies;
  r1.seg         = pl.seg.as<int2>();
  r1.lists       = p.lists.as<int>();
  r1.stride      = p.stride;
  r1.lr          = pl.lr;
  r1.sketch      = p.sketch.as<signed char>();
  r1.sketch_norm = p.sketch_norm.as<float>();
  r1.scale       = p.scale.as<float>();
  r1.qs          = pl.qs.as<float>();
  r1.sw          = sw;
  r1.vectors     = p.vectors.as<__half>();
  r1.D           = D;
  r1.Q           = pl.qbuf.as<float>();
  r1.R           = pl.R1;
  r1.KO          = pl.KO;
  r1.sketch_rank = sp.sketch_rank ? 1 : 0;
  r1.sketch_map  = map_of(ix, p.sketch_rows);
  r1.vector_map  = map_of(ix, p.vector_rows);
  r1.fresh       = 1;
  r1.si          = pl.si.as<long long>();
  r1.sd          = pl.sd.as<float>();
  r1.stats       = pl.stats.as<long long>();
  r1.phase       = pl.phase1.as<long long>();
  if (dbg.taps) {
    r1.tap_cand = pl.tap_cand.as<int>();
    r1.tap_dist = pl.tap_dist.as<float>();
    r1.tap_n    = pl.tap_n.as<int>();
    r1.tap_cap  = pl.tap_cap;
  }
  // sketch rows of this GPU's own memory (not the host tier, not dealt over GPUs) plus their constants
  const int64_t sketch_bytes = (p.sketch.host || p.sketch_rows.on) ? 0 : static_cast<int64_t>(p.sketch.size + p.sketch_norm.size);
  size_round(pl, r1, p.copies * pl.lr, 0, p.device, sketch_bytes);
  // waves: table rows of the start points
  if (sp.waves > 0) {
    auto& r2       = pl.r2;
    r2             = kernels::round_args{};
    r2.m           = pl.mw;
    r2.nseg        = S;
    r2.table       = p.table.as<int>();
    r2.table_len   = ix.table_len;
    r2.table_map   = map_of(ix, p.table_rows);
    r2.sketch_map  = r1.sketch_map;
    r2.vector_map  = r1.vector_map;
    r2.done        = pl.done.as<int>();
    r2.done_stride = S * sp.waves;
    r2.sketch      = r1.sketch;
    r2.sketch_norm = r1.sketch_norm;
    r2.scale       = r1.scale;
    r2.qs          = r1.qs + static_cast<size_t>(pl.lo - pl.q1) * sw;
    r2.sw          = sw;
    r2.vectors     = r1.vectors;
    r2.D           = D;
    r2.Q           = r1.Q + static_cast<size_t>(pl.lo - pl.q1) * D;
    r2.R           = pl.R2;
    r2.KO          = pl.KO;
    r2.sketch_rank = r1.sketch_rank;
    r2.fresh       = 0;
    r2.si          = pl.wsi;
    r2.sd          = pl.wsd;
    r2.stats       = r1.stats;
    r2.phase       = pl.phase2.as<long long>();
    size_round(pl, r2, S * ix.table_len, S * std::max(sp.waves - 1, 0), p.device, sketch_bytes);
  }
  kernels::round_allow_smem(pl.smem_max);

  // one eager run (module loading), then the capture (search.cu:754-786)
  OCTEX_CUDA_TRY(cudaDeviceSynchronize());
  run_batch(ix, pl, p.stream, nullptr);
  OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  check_tc(pl);
  OCTEX_CUDA_TRY(cudaEventCreateWithFlags(&pl.done_ev, cudaEventDisableTiming));
  // one graph per batch; with several processes the NCCL exchanges between the kernels are captured
  // into it too (every process replays its graph in the same order, as it would launch the calls)
  cudaGraph_t graph = nullptr;
  OCTEX_CUDA_TRY(cudaStreamBeginCapture(p.stream, cudaStreamCaptureModeThreadLocal));
  try {
    run_batch(ix, pl, p.stream, nullptr);
  } catch (...) {
    cudaStreamEndCapture(p.stream, &graph);
    if (graph != nullptr) cudaGraphDestroy(graph);
    throw;
  }
  OCTEX_CUDA_TRY(cudaStreamEndCapture(p.stream, &graph));
  OCTEX_CUDA_TRY(cudaGraphInstantiate(&pl.graph, graph, 0));
  OCTEX_CUDA_TRY(cudaGraphDestroy(graph));
  return plp;
}

auto get_plan(index_impl& ix, search_params const& sp, int m, int k, int lane) -> std::shared_ptr<plan>
{
  const debug_options dbg = ix_debug(ix);
  std::string key = std::to_string(m) + "/" + std::to_string(k) + "/" + std::to_string(sp.read) +
                    "/" + std::to_string(sp.starts) + "/" + std::to_string(sp.waves) + "/" +
                    std::to_string(sp.rerank) + "/" + std::to_string(sp.wave_rerank) + "/" +
                    std::to_string(sp.sketch_rank) + "/" + std::to_string(sp.final_rerank) + "/" +
                    std::to_string(dbg.stats) + std::to_string(dbg.taps) +
                    std::to_string(dbg.ordered_projection);
  std::lock_guard<std::mutex> lock(ix.mu);
  // one cached configuration: the previous buffers and graphs go before the new ones come
  // (search.cu:807-812); a configuration has one plan per lane (see search_impl)
  if (ix.plans.find(key) == ix.plans.end()) {
    ix.plans.clear();
    ix.plans[key] = make_plan(ix, sp, m, k, dbg);
  }
  if (lane == 0) return ix.plans[key];
  const std::string other = key + "#" + std::to_string(lane);
  auto it = ix.plans.find(other);
  if (it != ix.plans.end()) return it->second;
  auto pl          = make_plan(ix, sp, m, k, dbg);
  ix.plans[other]  = pl;
  return pl;
}

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
                 bool resident)
{
  auto& ix = idx.impl();
  OCTEX_EXPECTS(qdim == ix.dim, "octex: query dimension differs from the index");
  OCTEX_EXPECTS(k >= 1, "octex: k >= 1");
  if (nq == 0) return;
  int cur = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  cudaStream_t caller = res.stream;
  const int m         = static_cast<int>(std::min<int64_t>(std::max(sp.batch, 1), nq));
  auto pl             = get_plan(ix, sp, m, static_cast<int>(k));
  const int D = static_cast<int>(ix.dim);
  auto& p     = ix.part;
  // A call of several batches whose queries and results cross the bus alternates them between two
  // lanes, each a plan (buffers and graph) on a stream of its own: the copies of one batch run
  // under the kernels of the other. One lane when there is one batch, when the data is resident,
  // when processes exchange inside the batch (their collectives are ordered on one stream), and
  // when the plan keeps observations.
  const bool two_lanes = !resident && pl->world == 1 && nq > m && !pl->dbg.stats && !pl->dbg.taps;
  std::shared_ptr<plan> lane[2] = {pl, two_lanes ? get_plan(ix, sp, m, static_cast<int>(k), 1) : pl};
  std::unique_lock<std::mutex> lock0(lane[0]->mu), lock1;
  if (two_lanes) lock1 = std::unique_lock<std::mutex>(lane[1]->mu);
  if (two_lanes && p.second == nullptr) {
    OCTEX_CUDA_TRY(cudaSetDevice(p.device));
    OCTEX_CUDA_TRY(cudaStreamCreateWithFlags(&p.second, cudaStreamNonBlocking));
    OCTEX_CUDA_TRY(cudaSetDevice(cur));
  }
  cudaStream_t stream[2] = {p.stream, two_lanes ? p.second : p.stream};
  const int lanes        = two_lanes ? 2 : 1;
  // a search with device outputs returns before its kernels ran; had one of them given up, the
  // word is still set and this is the first host code to see it
  for (int l = 0; l < lanes; l++)
    check_tc(*lane[l]);

  // the work of this call starts after what the caller queued on its stream (search.cu:841-848)
  // an event of the plan (one search at a time uses it: pl->mu), on the device of the caller's
  // stream, which is the current one
  if (pl->start_ev == nullptr || pl->start_dev != cur) {
    if (pl->start_ev != nullptr) cudaEventDestroy(pl->start_ev);
    pl->start_ev = nullptr;
    OCTEX_CUDA_TRY(cudaEventCreateWithFlags(&pl->start_ev, cudaEventDisableTiming));
    pl->start_dev = cur;
  }
  cudaEvent_t start = pl->start_ev;
  OCTEX_CUDA_TRY(cudaEventRecord(start, caller));
  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  for (int l = 0; l < lanes; l++)
    OCTEX_CUDA_TRY(cudaStreamWaitEvent(stream[l], start, 0));
  int64_t batch = 0;
  for (int64_t b0 = 0; b0 < nq; b0 += m, batch++) {
    plan& w        = *lane[batch % lanes];
    cudaStream_t s = stream[batch % lanes];
    const int n    = static_cast<int>(std::min<int64_t>(m, nq - b0));
    if (!resident) {
      // rows [q1, q1 + m1) of the batch, the part beyond its end filled with copies of a row
      // (search.cu:870-883)
      int have = std::clamp(n - w.q1, 0, w.m1);
      if (have > 0) {
        OCTEX_CUDA_TRY(cudaMemcpyAsync(w.qbuf.ptr, queries + (b0 + w.q1) * D, sizeof(float) * have * D,
                                       cudaMemcpyDefault, s));
      } else if (w.m1 > 0) {
        OCTEX_CUDA_TRY(cudaMemcpyAsync(w.qbuf.ptr, queries + b0 * D, sizeof(float) * D, cudaMemcpyDefault, s));
        have = 1;
      }
      if (have < w.m1) kernels::pad_rows(w.qbuf.as<float>(), have, w.m1, D, s);
    }
    if (sp.use_graph && w.graph != nullptr)
      OCTEX_CUDA_TRY(cudaGraphLaunch(w.graph, s));
    else
      run_batch(ix, w, s, nullptr);  // use_graph = false, or a batch with exchanges
    if (!resident && w.world == 1) {
      OCTEX_CUDA_TRY(cudaMemcpyAsync(neighbors + b0 * k, w.bi, sizeof(int64_t) * n * k, cudaMemcpyDefault, s));
      OCTEX_CUDA_TRY(cudaMemcpyAsync(distances + b0 * k, w.bd, sizeof(float) * n * k, cudaMemcpyDefault, s));
    } else if (!resident) {
      // the gathered results: block r holds the rows [lo_r, hi_r) of the batch
      for (int r = 0; r < w.world; r++) {
        const int lo_r = static_cast<int>(int64_t{m} * r / w.world);
        const int hi_r = static_cast<int>(int64_t{m} * (r + 1) / w.world);
        const int rows = std::clamp(n - lo_r, 0, hi_r - lo_r);
        if (rows == 0) continue;
        const char* block = w.gathered.as<char>() + static_cast<size_t>(r) * w.out_block;
        OCTEX_CUDA_TRY(cudaMemcpyAsync(neighbors + (b0 + lo_r) * k, block, sizeof(int64_t) * rows * k,
                                       cudaMemcpyDefault, s));
        OCTEX_CUDA_TRY(cudaMemcpyAsync(distances + (b0 + lo_r) * k, block + w.out_ids, sizeof(float) * rows * k,
                                       cudaMemcpyDefault, s));
      }
    }
  }
  for (int l = 0; l < lanes; l++)
    OCTEX_CUDA_TRY(cudaEventRecord(lane[l]->done_ev, stream[l]));
  OCTEX_CUDA_TRY(cudaSetDevice(cur));
  for (int l = 0; l < lanes; l++)
    OCTEX_CUDA_TRY(cudaStreamWaitEvent(caller, lane[l]->done_ev, 0));
  if (host_out) OCTEX_CUDA_TRY(cudaStreamSynchronize(caller));
  if (host_out)
    for (int l = 0; l < lanes; l++)
      check_tc(*lane[l]);
}

}  // namespace detail

void search(resources const& res, search_params const& params, index const& idx,
            host_matrix_view<const float> queries, host_matrix_view<int64_t> neighbors,
            host_matrix_view<float> distances)
{
  OCTEX_EXPECTS(neighbors.rows == queries.rows && distances.rows == queries.rows &&
                  distances.cols == neighbors.cols,
                "octex: output shapes");
  detail::search_impl(res, params, idx, queries.data, queries.rows, queries.cols, neighbors.data,
                      distances.data, neighbors.cols, true, false);
}

void search(resources const& res, search_params const& params, index const& idx,
            device_matrix_view<const float> queries, device_matrix_view<int64_t> neighbors,
            device_matrix_view<float> distances)
{
  OCTEX_EXPECTS(neighbors.rows == queries.rows && distances.rows == queries.rows &&
                  distances.cols == neighbors.cols,
                "octex: output shapes");
  detail::search_impl(res, params, idx, queries.data, queries.rows, queries.cols, neighbors.data,
                      distances.data, neighbors.cols, false, false);
}

}  // namespace octex_b200
