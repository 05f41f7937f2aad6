// Index directory (or arrays in memory) -> arrays placed on this process's GPU.
//
// Answers cpp/src/neighbors/octex/load.cu:206-494 of hpdic/octex for one process per GPU: the
// parameter checks, the dealing of copies (shard: equal consecutive ranges over the processes, or
// saved parts round robin; replicate: all), list truncation to list_limit, and the operand
// preparation of the projection (fp16, here K-major for the tensor-core kernel) are the same.

#include "index_impl.hpp"
#include "kernels.hpp"
#include "npy.hpp"

#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstring>

namespace octex_b200 {

namespace detail {

index_impl::~index_impl()
{
  plans.clear();
}

namespace {

/// Host memory -> device through two pinned buffers; device memory -> device directly.
class stager {
 public:
  stager(int device, cudaStream_t s) : stream_(s)
  {
    OCTEX_CUDA_TRY(cudaSetDevice(device));
    for (int i = 0; i < 2; i++) {
      OCTEX_CUDA_TRY(cudaHostAlloc(&pin_[i], kChunk, cudaHostAllocDefault));
      OCTEX_CUDA_TRY(cudaEventCreateWithFlags(&ev_[i], cudaEventDisableTiming));
    }
  }
  stager(stager const&) = delete;
  ~stager()
  {
    for (int i = 0; i < 2; i++) {
      if (ev_[i] != nullptr) cudaEventDestroy(ev_[i]);
      if (pin_[i] != nullptr) cudaFreeHost(pin_[i]);
    }
  }
  void copy(void* dst, const void* src, size_t bytes)
  {
    if (bytes == 0) return;
    cudaPointerAttributes at{};
    cudaError_t e = cudaPointerGetAttributes(&at, src);
    if (e != cudaSuccess) cudaGetLastError();
    if (e == cudaSuccess && (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged ||
                             at.type == cudaMemoryTypeHost)) {
      OCTEX_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream_));
      if (at.type == cudaMemoryTypeHost) OCTEX_CUDA_TRY(cudaStreamSynchronize(stream_));
      return;
    }
    auto* d = static_cast<char*>(dst);
    auto* s = static_cast<const char*>(src);
    for (size_t o = 0; o < bytes; o += kChunk) {
      const size_t nb = std::min(kChunk, bytes - o);
      OCTEX_CUDA_TRY(cudaEventSynchronize(ev_[turn_]));
      std::memcpy(pin_[turn_], s + o, nb);
      OCTEX_CUDA_TRY(cudaMemcpyAsync(d + o, pin_[turn_], nb, cudaMemcpyHostToDevice, stream_));
      OCTEX_CUDA_TRY(cudaEventRecord(ev_[turn_], stream_));
      turn_ ^= 1;
    }
  }
  /// Bring `bytes` at src (host or device) into host memory.
  void fetch(void* dst, const void* src, size_t bytes)
  {
    if (bytes == 0) return;
    cudaPointerAttributes at{};
    cudaError_t e = cudaPointerGetAttributes(&at, src);
    if (e != cudaSuccess) cudaGetLastError();
    if (e == cudaSuccess && (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged)) {
      OCTEX_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream_));
      OCTEX_CUDA_TRY(cudaStreamSynchronize(stream_));
    } else {
      std::memcpy(dst, src, bytes);
    }
  }

 private:
  static constexpr size_t kChunk = size_t{64} << 20;
  cudaStream_t stream_;
  void* pin_[2]        = {nullptr, nullptr};
  cudaEvent_t ev_[2]   = {nullptr, nullptr};
  int turn_            = 0;
};

auto is_device_pointer(const void* p) -> bool
{
  cudaPointerAttributes at{};
  cudaError_t e = cudaPointerGetAttributes(&at, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

}  // namespace

void place(index_impl& ix, source_arrays const& src)
{
  auto const& a      = src.a;
  auto const& params = ix.params;
  const int L        = static_cast<int>(ix.spacings.size());
  const int width    = 8 * ix.blocks;
  const int64_t D = ix.dim, N = ix.n, S = ix.sketch_width;
  const int64_t T1 = (int64_t{1} << ix.log_buckets) + 1;
  OCTEX_EXPECTS(ix.dim % 2 == 0, "octex: the dimension must be even");
  OCTEX_EXPECTS(ix.dim <= kernels::kMaxDim,
                "octex: dimensions above " + std::to_string(kernels::kMaxDim) + " are not supported");
  OCTEX_EXPECTS(ix.sketch_width % 16 == 0 && ix.sketch_width <= 512 && ix.sketch_width > 0,
                "octex: sketch width: a multiple of 16, <= 512");
  OCTEX_EXPECTS((ix.blocks >= 1 && ix.blocks <= 6) || ix.blocks == 8,
                "octex: blocks must be 1-6 or 8");
  OCTEX_EXPECTS(L >= 1 && L <= 16, "octex: 1 to 16 spacings");
  OCTEX_EXPECTS(ix.log_buckets >= 1 && ix.log_buckets <= 30, "octex: log_buckets in [1, 30]");
  OCTEX_EXPECTS(ix.world >= 1 && ix.rank >= 0 && ix.rank < ix.world, "octex: rank outside world");

  // copies of this process (load.cu:252-281)
  const int all    = src.all_copies;
  const int nparts = std::max(1, params.parts);
  std::vector<std::vector<int>> part_copies(nparts);
  ix.copies = 0;
  for (int q = 0; q < nparts; q++) {
    int lo = static_cast<int>(int64_t{all} * q / nparts);
    int hi = static_cast<int>(int64_t{all} * (q + 1) / nparts);
    if (params.copies_per_part > 0) hi = std::min(hi, lo + params.copies_per_part);
    if (nparts == 1 && params.copies_limit > 0) hi = std::min(hi, lo + params.copies_limit);
    for (int c = lo; c < hi; c++)
      part_copies[q].push_back(c);
    ix.copies += static_cast<int>(part_copies[q].size());
  }
  const bool shard = params.mode == placement::shard && ix.world > 1;
  std::vector<int> cl;
  if (!shard) {
    for (auto const& pc : part_copies)
      cl.insert(cl.end(), pc.begin(), pc.end());
  } else if (nparts == 1) {
    auto const& pc = part_copies[0];
    cl.assign(pc.begin() + pc.size() * ix.rank / ix.world,
              pc.begin() + pc.size() * (ix.rank + 1) / ix.world);
  } else {
    for (int q = ix.rank; q < nparts; q += ix.world)
      cl.insert(cl.end(), part_copies[q].begin(), part_copies[q].end());
  }
  OCTEX_EXPECTS(!cl.empty(), "octex: a device holds no copies (fewer copies or parts than devices)");

  auto& p  = ix.part;
  p.device = ix.devices.at(0);
  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  OCTEX_CUDA_TRY(cudaStreamCreateWithFlags(&p.stream, cudaStreamNonBlocking));
  stager st(p.device, p.stream);
  p.copy0      = cl.front();
  p.copies     = static_cast<int>(cl.size());
  const int Cg = p.copies;
  const bool whole = Cg == all && cl.front() == 0;  // every copy, in order
  const int ll = params.list_limit > 0 ? std::min(params.list_limit, ix.list_len) : ix.list_len;

  auto own = [&](dbuf& dst, size_t bytes) {
    dst = dbuf(p.device, bytes);
    p.bytes += static_cast<int64_t>(bytes);
  };
  // runs of consecutive copies, per_copy bytes each, into the device array in list order; arrays
  // already on this device and wanted whole are used in place when the caller allows it
  auto put = [&](dbuf& dst, const void* srcp, size_t per_copy) {
    if (a.borrow && whole && is_device_pointer(srcp)) {
      dst = dbuf::borrow(p.device, srcp, per_copy * Cg);
      return;
    }
    own(dst, per_copy * Cg);
    for (int i = 0; i < Cg;) {
      int j = i + 1;
      while (j < Cg && cl[j] == cl[j - 1] + 1)
        j++;
      st.copy(dst.as<char>() + per_copy * i, static_cast<const char*>(srcp) + per_copy * cl[i],
              per_copy * (j - i));
      i = j;
    }
  };
  auto put_rows = [&](dbuf& dst, const void* srcp, size_t bytes) {
    if (a.borrow && is_device_pointer(srcp)) {
      dst = dbuf::borrow(p.device, srcp, bytes);
      return;
    }
    own(dst, bytes);
    st.copy(dst.ptr, srcp, bytes);
  };
  // the host tier (load.cu:328-330): the array lives in page-locked host memory and the kernels
  // read it over the bus through the same pointer; it does not count as device memory
  auto put_rows_host = [&](dbuf& dst, const void* srcp, size_t bytes) {
    dst = dbuf::pinned(p.device, bytes);
    OCTEX_CUDA_TRY(cudaMemcpyAsync(dst.ptr, srcp, bytes, cudaMemcpyDefault, p.stream));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  };

  // lists: the first ll entries of every cell row (load.cu:361-379)
  const int64_t stride0 = a.stride;
  if (ll == ix.list_len) {
    p.stride = stride0;
    put(p.lists, a.lists, static_cast<size_t>(stride0) * sizeof(int32_t));
  } else {
    const int64_t rows = stride0 / ix.list_len;
    p.stride           = rows * ll;
    own(p.lists, static_cast<size_t>(Cg * p.stride) * sizeof(int32_t));
    std::vector<int32_t> full(stride0), cut(p.stride);
    for (int c = 0; c < Cg; c++) {
      st.fetch(full.data(), a.lists + int64_t{cl[c]} * stride0, stride0 * sizeof(int32_t));
      for (int64_t r = 0; r < rows; r++)
        std::memcpy(cut.data() + r * ll, full.data() + r * ix.list_len, ll * sizeof(int32_t));
      st.copy(p.lists.as<int32_t>() + c * p.stride, cut.data(), p.stride * sizeof(int32_t));
      OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));  // cut is reused
    }
  }
  p.mmax = a.mmax;
  put(p.base, a.base, static_cast<size_t>(L) * sizeof(int32_t));

  // The cells of every (copy, level). The directory holds them as CSR bucket bounds over sorted
  // keys (offsets [C, L, T + 1], keys [C, L, mmax]: build.cu:215-349 of the reference); the kernels
  // here look them up in one open-addressing table per (copy, level), slot = (key, row of the
  // cell), at most half full, built on the GPU from the keys. The last CSR bound of a level is its
  // cell count; the bucket bounds themselves never go to the GPU.
  {
    const int CL = Cg * L;
    std::vector<int> ncells(CL), mask(CL);
    std::vector<long long> off(CL);
    std::vector<unsigned char> on(static_cast<size_t>(CL));
    long long slots = 0;
    for (int c = 0; c < Cg; c++)
      for (int j = 0; j < L; j++) {
        int32_t last = 0;
        st.fetch(&last, a.offsets + (int64_t{cl[c]} * L + j) * T1 + (T1 - 1), sizeof(int32_t));
        OCTEX_EXPECTS(last >= 0 && last <= p.mmax, "octex: a level's cell count exceeds its key array");
        const int k = c * L + j;
        ncells[k]   = last;
        on[k]       = last > 0;
        int cap     = 4;
        while (cap < 2 * last)
          cap <<= 1;
        mask[k] = cap - 1;
        off[k]  = slots;
        slots += cap;
      }
    own(p.level_on, on.size());
    st.copy(p.level_on.ptr, on.data(), on.size());
    own(p.cell_off, sizeof(long long) * CL);
    st.copy(p.cell_off.ptr, off.data(), p.cell_off.size);
    own(p.cell_mask, sizeof(int) * CL);
    st.copy(p.cell_mask.ptr, mask.data(), p.cell_mask.size);
    own(p.cell_table, sizeof(kernels::cell_slot) * static_cast<size_t>(slots));
    OCTEX_CUDA_TRY(cudaMemsetAsync(p.cell_table.ptr, 0xff, p.cell_table.size, p.stream));
    // the keys of this process's copies on the GPU for the duration of the build
    dbuf keys, counts(p.device, sizeof(int) * CL);
    const int64_t before = p.bytes;
    put(keys, a.keys, static_cast<size_t>(L) * p.mmax * sizeof(int64_t));
    p.bytes = before;  // not kept
    st.copy(counts.ptr, ncells.data(), counts.size);
    kernels::build_cell_tables(keys.as<long long>(), p.mmax, counts.as<int>(), p.cell_off.as<long long>(),
                               p.cell_mask.as<int>(), CL, p.cell_table.as<kernels::cell_slot>(), p.stream);
    OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  }

  // projections, one K-major fp16 row per projected coordinate, and shifts (load.cu:385-402)
  p.ldu = static_cast<int>((D + 63) / 64 * 64);
  {
    std::vector<float> pr(static_cast<size_t>(D) * width), sh(width);
    std::vector<__half> ut(static_cast<size_t>(Cg) * width * p.ldu, __float2half(0.f)),
      hs(static_cast<size_t>(Cg) * width);
    for (int c = 0; c < Cg; c++) {
      st.fetch(pr.data(), a.proj + int64_t{cl[c]} * D * width, pr.size() * sizeof(float));
      st.fetch(sh.data(), a.shift + int64_t{cl[c]} * width, sh.size() * sizeof(float));
      for (int64_t d = 0; d < D; d++)
        for (int s = 0; s < width; s++)
          ut[(static_cast<size_t>(c) * width + s) * p.ldu + d] = __float2half(pr[d * width + s]);
      for (int s = 0; s < width; s++)
        hs[c * width + s] = __float2half(sh[s]);
    }
    std::vector<float> inv(L);
    for (int j = 0; j < L; j++)
      inv[j] = static_cast<float>(1.0 / static_cast<double>(ix.spacings[j]));
    own(p.ut, ut.size() * sizeof(__half));
    st.copy(p.ut.ptr, ut.data(), p.ut.size);
    own(p.shift, hs.size() * sizeof(__half));
    st.copy(p.shift.ptr, hs.data(), p.shift.size);
    own(p.inv_f, inv.size() * sizeof(float));
    st.copy(p.inv_f.ptr, inv.data(), p.inv_f.size);
    OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  }
  own(p.mean, D * sizeof(float));
  st.copy(p.mean.ptr, a.mean, p.mean.size);
  own(p.basis, D * S * sizeof(float));
  st.copy(p.basis.ptr, a.basis, p.basis.size);
  own(p.scale, S * sizeof(float));
  st.copy(p.scale.ptr, a.scale, p.scale.size);
  // rows dealt over the processes (load.cu:315,406-427): this process keeps rows
  // [rank * rows_per, (rank + 1) * rows_per) in memory of its own; the other ranges are mapped in
  // when the processes connect. With one process every array is whole.
  const int64_t rows_per = (N + ix.world - 1) / ix.world;
  auto put_rows_dealt    = [&](dbuf& dst, dealt_rows& d, const void* srcp, size_t row_bytes) {
    d.on             = true;
    d.rows_per       = rows_per;
    d.row0           = std::min<int64_t>(N, ix.rank * rows_per);
    const int64_t r1 = std::min<int64_t>(N, d.row0 + rows_per);
    own(dst, static_cast<size_t>(r1 - d.row0) * row_bytes);
    st.copy(dst.ptr, static_cast<const char*>(srcp) + d.row0 * row_bytes, dst.size);
  };
  const bool many = ix.world > 1;
  if (params.sketch == sketch_placement::host)
    put_rows_host(p.sketch, a.sketch, static_cast<size_t>(N * S));
  else if (params.sketch == sketch_placement::shard && many)
    put_rows_dealt(p.sketch, p.sketch_rows, a.sketch, static_cast<size_t>(S));
  else
    put_rows(p.sketch, a.sketch, static_cast<size_t>(N * S));
  // The constant of every sketch row (kernels::sketch_row_norms), 4 bytes per row, on this GPU for
  // all rows whatever tier or process holds the codes: the rows pass through the GPU in chunks.
  {
    own(p.sketch_norm, static_cast<size_t>(N) * sizeof(float));
    const int64_t chunk = std::max<int64_t>(1, (int64_t{256} << 20) / S);
    dbuf raw(p.device, static_cast<size_t>(std::min(chunk, N) * S));
    for (int64_t r = 0; r < N; r += chunk) {
      const int64_t nr = std::min(chunk, N - r);
      st.copy(raw.ptr, a.sketch + r * S, static_cast<size_t>(nr * S));
      kernels::sketch_row_norms(raw.as<signed char>(), p.scale.as<float>(), nr, static_cast<int>(S),
                                p.sketch_norm.as<float>() + r, p.stream);
      OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));  // raw is reused
    }
  }
  if (params.vectors_on_host)
    put_rows_host(p.vectors, a.vectors, static_cast<size_t>(N * D) * sizeof(__half));
  else if (params.shard_vectors && many)
    put_rows_dealt(p.vectors, p.vector_rows, a.vectors, static_cast<size_t>(D) * sizeof(__half));
  else
    put_rows(p.vectors, a.vectors, static_cast<size_t>(N * D) * sizeof(__half));
  if (ix.table_len > 0) {
    OCTEX_EXPECTS(a.table != nullptr, "octex: table_len > 0 without a table");
    if (params.table_on_host)
      put_rows_host(p.table, a.table, static_cast<size_t>(N * ix.table_len) * sizeof(int32_t));
    else if (shard)  // shard placement always deals the table (load.cu:421-427)
      put_rows_dealt(p.table, p.table_rows, a.table, static_cast<size_t>(ix.table_len) * sizeof(int32_t));
    else
      put_rows(p.table, a.table, static_cast<size_t>(N * ix.table_len) * sizeof(int32_t));
  }
  OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  ix.list_len = ll;
}

/// Once the processes have a communicator: every process publishes the address of the row ranges
/// it holds and maps the other processes' ranges into its own address space (CUDA IPC handles,
/// exchanged with an all-gather); the kernels then read a row wherever it lives with plain loads,
/// as the reference's kernels do through its xptr / cptr / tptr tables (load.cu:187-202,444-490).
void connect_rows(index_impl& ix)
{
  auto& p = ix.part;
  if (ix.world <= 1 || ix.comm == nullptr) return;
  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  struct item {
    dealt_rows* d;
    dbuf* mine;
  };
  const item items[] = {{&p.table_rows, &p.table}, {&p.sketch_rows, &p.sketch}, {&p.vector_rows, &p.vectors}};
  const size_t hb = sizeof(cudaIpcMemHandle_t);
  dbuf send(p.device, hb), recv(p.device, hb * ix.world);
  for (auto const& it : items) {
    auto& d = *it.d;
    if (!d.on || d.ptrs.ptr != nullptr) continue;
    cudaIpcMemHandle_t h{};
    if (it.mine->size != 0) OCTEX_CUDA_TRY(cudaIpcGetMemHandle(&h, it.mine->ptr));
    OCTEX_CUDA_TRY(cudaMemcpyAsync(send.ptr, &h, hb, cudaMemcpyHostToDevice, p.stream));
    ix.comm->all_gather(send.ptr, recv.ptr, hb, p.stream);
    std::vector<cudaIpcMemHandle_t> all(ix.world);
    OCTEX_CUDA_TRY(cudaMemcpyAsync(all.data(), recv.ptr, hb * ix.world, cudaMemcpyDeviceToHost, p.stream));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
    std::vector<long long> ptrs(ix.world, 0);
    for (int g = 0; g < ix.world; g++) {
      const int64_t r0 = std::min<int64_t>(ix.n, g * d.rows_per);
      const int64_t r1 = std::min<int64_t>(ix.n, r0 + d.rows_per);
      if (r1 <= r0) continue;  // that process holds no rows
      if (g == ix.rank) {
        ptrs[g] = reinterpret_cast<long long>(it.mine->ptr);
      } else {
        void* q = nullptr;
        OCTEX_CUDA_TRY(cudaIpcOpenMemHandle(&q, all[g], cudaIpcMemLazyEnablePeerAccess));
        d.opened.push_back(q);
        ptrs[g] = reinterpret_cast<long long>(q);
      }
    }
    d.ptrs = dbuf(p.device, sizeof(long long) * ix.world);
    OCTEX_CUDA_TRY(cudaMemcpyAsync(d.ptrs.ptr, ptrs.data(), d.ptrs.size, cudaMemcpyHostToDevice, p.stream));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  }
  std::lock_guard<std::mutex> lock(ix.mu);
  ix.plans.clear();  // plans made before the connection do not know the tables
}

void set_table(index_impl& ix, const int32_t* table, int table_len)
{
  OCTEX_EXPECTS(ix.world == 1, "octex: the table of an index shared by several processes cannot be replaced");
  OCTEX_EXPECTS(table_len >= 0 && (table_len == 0 || table != nullptr), "octex: set_table needs a table");
  auto& p = ix.part;
  {
    std::lock_guard<std::mutex> lock(ix.mu);
    ix.plans.clear();
  }
  int cur = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  if (!p.table.host) p.bytes -= static_cast<int64_t>(p.table.size);
  p.table      = dbuf();
  p.table_rows = dealt_rows{};
  ix.table_len = table_len;
  if (table_len > 0) {
    p.table = dbuf(p.device, static_cast<size_t>(ix.n) * table_len * sizeof(int32_t));
    p.bytes += static_cast<int64_t>(p.table.size);
    OCTEX_CUDA_TRY(cudaMemcpyAsync(p.table.ptr, table, p.table.size, cudaMemcpyDefault, p.stream));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  }
  OCTEX_CUDA_TRY(cudaSetDevice(cur));
}

void disconnect_rows(index_impl& ix)
{
  auto& p = ix.part;
  if (ix.world <= 1 || ix.comm == nullptr) return;
  OCTEX_CUDA_TRY(cudaSetDevice(p.device));
  {
    std::lock_guard<std::mutex> lock(ix.mu);
    ix.plans.clear();  // their graphs hold the exchanges and the addresses of the mapped ranges
  }
  OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  for (dealt_rows* d : {&p.table_rows, &p.sketch_rows, &p.vector_rows}) {
    for (void* q : d->opened)
      OCTEX_CUDA_TRY(cudaIpcCloseMemHandle(q));
    d->opened.clear();
    d->ptrs = dbuf();
  }
  // nobody frees an exported range before everybody has unmapped it
  dbuf one(p.device, 1), all(p.device, static_cast<size_t>(ix.world));
  ix.comm->all_gather(one.ptr, all.ptr, 1, p.stream);
  OCTEX_CUDA_TRY(cudaStreamSynchronize(p.stream));
  ix.comm.reset();
}

}  // namespace detail

index::index(std::shared_ptr<detail::index_impl> impl) : impl_(std::move(impl)) {}
index::index(index&&) noexcept                    = default;
auto index::operator=(index&&) noexcept -> index& = default;
index::~index()                                   = default;
auto index::size() const noexcept -> int64_t { return impl_->n; }
auto index::dim() const noexcept -> int64_t { return impl_->dim; }
auto index::copies() const noexcept -> int { return impl_->copies; }
auto index::devices() const noexcept -> std::vector<int> const& { return impl_->devices; }
auto index::device_bytes() const -> std::vector<int64_t> { return {impl_->part.bytes}; }
auto index::impl() const noexcept -> detail::index_impl& { return *impl_; }

namespace {

void choose_device(detail::index_impl& ix, load_params const& params, bool from_directory)
{
  OCTEX_EXPECTS(params.mode == placement::replicate || params.mode == placement::shard,
                "octex: placement must be replicate or shard");
  int cur = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  if (params.devices.empty()) {
    // The reference places an index on every visible GPU when none is named
    // (cpp/src/neighbors/octex/load.cu:241-251). This library drives one GPU per process, so a
    // caller of the reference's load on a machine with several GPUs must say which one it means
    // rather than silently get one of them; a process that states its rank among several
    // (load_params::world > 1) has said so.
    int visible = 1;
    OCTEX_CUDA_TRY(cudaGetDeviceCount(&visible));
    OCTEX_EXPECTS(!from_directory || visible <= 1 || params.world > 1,
                  "octex: " + std::to_string(visible) +
                    " GPUs are visible and load_params::devices names none: this library drives one "
                    "GPU per process; name the device (devices = {d}), or start one process per GPU "
                    "and give each its rank and world");
    ix.devices = {cur};
  } else {
    OCTEX_EXPECTS(params.devices.size() == 1,
                  "octex: one process drives one GPU here; start one process per device and give "
                  "each its rank (load_params::rank / world)");
    ix.devices = params.devices;
  }
  ix.rank  = params.rank;
  ix.world = std::max(1, params.world);
}

}  // namespace

auto load(resources const& res, std::string const& path, load_params const& params) -> index
{
  (void)res;
  auto impl = std::make_shared<detail::index_impl>();
  auto& ix  = *impl;
  ix.path   = path;
  ix.params = params;
  const std::string text = read_text(path + "/meta.json");
  json_value meta        = json_reader(text).parse();
  OCTEX_EXPECTS(static_cast<int>(meta.num("format", 1)) == 1, "octex: unknown index format");
  ix.n            = static_cast<int64_t>(meta.num("n", 0));
  ix.dim          = static_cast<int64_t>(meta.num("dim", 0));
  ix.blocks       = static_cast<int>(meta.num("blocks", 4));
  ix.list_len     = static_cast<int>(meta.num("list_len", 0));
  ix.log_buckets  = static_cast<int>(meta.num("log_buckets", 20));
  ix.sketch_width = static_cast<int>(meta.num("sketch_width", 0));
  ix.table_len    = static_cast<int>(meta.num("table_len", 0));
  if (meta.has("spacings"))
    for (auto const& v : meta.at("spacings").items)
      ix.spacings.push_back(static_cast<float>(v.number));
  if (meta.has("metric"))
    OCTEX_EXPECTS(meta.at("metric").text == "sqeuclidean", "octex: the metric must be sqeuclidean");
  auto file = [&](std::string const& name) -> std::string {
    if (meta.has("files") && meta.at("files").has(name)) {
      std::string const& f = meta.at("files").at(name).text;
      return (!f.empty() && f[0] == '/') ? f : path + "/" + f;
    }
    return path + "/" + name + ".npy";
  };
  choose_device(ix, params, true);

  npy_file lists(file("lists")), keys(file("keys")), offsets(file("offsets")), base(file("base"));
  npy_file proj(file("proj")), shift(file("shift")), mean(file("mean"));
  npy_file basis(file("sketch_basis")), scale(file("sketch_scale")), sketch(file("sketch"));
  npy_file vectors(file("vectors"));
  std::unique_ptr<npy_file> table;
  if (ix.table_len > 0) table = std::make_unique<npy_file>(file("table"));
  lists.expect("<i4", 2, "lists");
  keys.expect("<i8", 3, "keys");
  offsets.expect("<i4", 3, "offsets");
  base.expect("<i4", 2, "base");
  proj.expect("<f4", 3, "proj");
  shift.expect("<f4", 2, "shift");
  mean.expect("<f4", 1, "mean");
  basis.expect("<f4", 2, "sketch_basis");
  scale.expect("<f4", 1, "sketch_scale");
  sketch.expect("|i1", 2, "sketch");
  vectors.expect("<f2", 2, "vectors");
  if (table) table->expect("<i4", 2, "table");

  const int all = static_cast<int>(meta.num("copies", 0));
  const int L   = static_cast<int>(ix.spacings.size());
  OCTEX_EXPECTS(lists.shape[0] == all && keys.shape[0] == all && keys.shape[1] == L &&
                  offsets.shape[0] == all && offsets.shape[1] == L &&
                  offsets.shape[2] == (int64_t{1} << ix.log_buckets) + 1 &&
                  proj.shape[0] == all && proj.shape[1] == ix.dim &&
                  proj.shape[2] == 8 * ix.blocks && base.shape[0] == all && base.shape[1] == L,
                "octex: bad shapes");
  OCTEX_EXPECTS(vectors.shape[0] == ix.n && vectors.shape[1] == ix.dim, "octex: vectors shape");
  OCTEX_EXPECTS(sketch.shape[0] == ix.n && sketch.shape[1] == ix.sketch_width &&
                  basis.shape[0] == ix.dim && basis.shape[1] == ix.sketch_width,
                "octex: sketch shape");
  OCTEX_EXPECTS(!table || (table->shape[0] == ix.n && table->shape[1] == ix.table_len),
                "octex: table shape");

  detail::source_arrays src;
  src.all_copies = all;
  auto& a        = src.a;
  a.stride       = lists.shape[1];
  a.mmax         = keys.shape[2];
  a.mean         = mean.as<float>();
  a.proj         = proj.as<float>();
  a.shift        = shift.as<float>();
  a.lists        = lists.as<int32_t>();
  a.keys         = keys.as<int64_t>();
  a.offsets      = offsets.as<int32_t>();
  a.base         = base.as<int32_t>();
  a.basis        = basis.as<float>();
  a.scale        = scale.as<float>();
  a.sketch       = sketch.as<int8_t>();
  a.vectors      = vectors.data;
  a.table        = table ? table->as<int32_t>() : nullptr;
  int cur        = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  detail::place(ix, src);
  OCTEX_CUDA_TRY(cudaSetDevice(cur));
  return index(impl);
}

auto attach(resources const& res, index_arrays const& arrays, load_params const& params) -> index
{
  (void)res;
  auto impl = std::make_shared<detail::index_impl>();
  auto& ix  = *impl;
  ix.params = params;
  ix.n            = arrays.n;
  ix.dim          = arrays.dim;
  ix.blocks       = arrays.blocks;
  ix.list_len     = arrays.list_len;
  ix.log_buckets  = arrays.log_buckets;
  ix.sketch_width = arrays.sketch_width;
  ix.table_len    = arrays.table_len;
  ix.spacings     = arrays.spacings;
  OCTEX_EXPECTS(arrays.mean && arrays.proj && arrays.shift && arrays.lists && arrays.keys &&
                  arrays.offsets && arrays.base && arrays.basis && arrays.scale && arrays.sketch &&
                  arrays.vectors,
                "octex: an index array is missing");
  choose_device(ix, params, false);
  detail::source_arrays src;
  src.a          = arrays;
  src.all_copies = arrays.copies;
  int cur        = 0;
  OCTEX_CUDA_TRY(cudaGetDevice(&cur));
  detail::place(ix, src);
  OCTEX_CUDA_TRY(cudaSetDevice(cur));
  return index(impl);
}

}  // namespace octex_b200
