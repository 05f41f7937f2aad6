// C boundary: parameter structs, index handle, load, search, and the cuVS-style resources and
// error text they lean on. Conventions follow the reference's C layer (hpdic/octex,
// c/src/neighbors/octex.cpp and c/src/core/exceptions.hpp:17-33, interop.hpp:51-97): every C++
// exception becomes CUVS_ERROR plus a per-thread message, cleared on success; argument checks
// that need no GPU work with res == 0.

#include "build.hpp"
#include "search_impl.hpp"

#include <octex_b200.h>
#include <octex_b200.hpp>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

template <typename F>
auto translate(F&& body) -> cuvsError_t
{
  try {
    body();
    g_last_error.clear();
    return CUVS_SUCCESS;
  } catch (std::exception const& e) {
    g_last_error = e.what();
    return CUVS_ERROR;
  } catch (...) {
    g_last_error = "octex: unknown error";
    return CUVS_ERROR;
  }
}

struct resources_box {
  octex_b200::resources res;
};

auto as_res(cuvsResources_t r) -> octex_b200::resources
{
  if (r == 0) return octex_b200::resources{};
  return reinterpret_cast<resources_box*>(r)->res;
}

auto to_cpp(cuvsOctexLoadParams const& p) -> octex_b200::load_params
{
  OCTEX_EXPECTS(p.placement == OCTEX_PLACEMENT_REPLICATE || p.placement == OCTEX_PLACEMENT_SHARD,
                "octex: unknown placement");
  OCTEX_EXPECTS(p.sketch == OCTEX_SKETCH_REPLICATE || p.sketch == OCTEX_SKETCH_SHARD ||
                  p.sketch == OCTEX_SKETCH_HOST,
                "octex: unknown sketch placement");
  octex_b200::load_params out;
  if (p.devices != nullptr && p.n_devices > 0) out.devices.assign(p.devices, p.devices + p.n_devices);
  out.mode            = static_cast<octex_b200::placement>(static_cast<int>(p.placement));
  out.vectors_on_host = p.vectors_on_host;
  out.shard_vectors   = p.shard_vectors;
  out.table_on_host   = p.table_on_host;
  out.sketch          = static_cast<octex_b200::sketch_placement>(static_cast<int>(p.sketch));
  out.parts           = p.parts;
  out.copies_per_part = p.copies_per_part;
  out.copies_limit    = p.copies_limit;
  out.list_limit      = p.list_limit;
  return out;
}

auto to_cpp(cuvsOctexSearchParams const& p) -> octex_b200::search_params
{
  octex_b200::search_params out;
  out.read            = p.read;
  out.starts          = p.starts;
  out.waves           = p.waves;
  out.rerank          = p.rerank;
  out.wave_rerank     = p.wave_rerank;
  out.batch           = p.batch;
  out.sketch_rank     = p.sketch_rank;
  out.final_rerank    = p.final_rerank;
  out.balanced_gather = p.balanced_gather;
  out.fused_merge     = p.fused_merge;
  out.use_graph       = p.use_graph;
  return out;
}

auto as_index(cuvsOctexIndex const& index) -> octex_b200::index*
{
  OCTEX_EXPECTS(index.addr != 0, "octex: the index is empty (load it first)");
  return reinterpret_cast<octex_b200::index*>(index.addr);
}

/// Report (once) a kernel of the last batches that gave up; the stream of the index is idle.
void check_last(octex_b200::detail::index_impl& ix)
{
  std::vector<std::shared_ptr<octex_b200::detail::plan>> plans;
  {
    std::lock_guard<std::mutex> lock(ix.mu);
    for (auto const& kv : ix.plans)
      plans.push_back(kv.second);
  }
  for (auto const& pl : plans)
    octex_b200::detail::check_tc(*pl);
}

template <typename T>
struct dl_code;
template <>
struct dl_code<float> {
  static constexpr int value = kDLFloat;
};
template <>
struct dl_code<int64_t> {
  static constexpr int value = kDLInt;
};

/// A dense row-major matrix of T out of a DLPack tensor (interop.hpp:51-97).
template <typename T>
auto matrix_of(DLManagedTensor* mt, bool on_device, T** data, int64_t* rows, int64_t* cols) -> void
{
  OCTEX_EXPECTS(mt != nullptr, "octex: a tensor is NULL");
  DLTensor const& t = mt->dl_tensor;
  const auto dev    = t.device.device_type;
  if (on_device)
    OCTEX_EXPECTS(dev == kDLCUDA || dev == kDLCUDAManaged || dev == kDLCUDAHost,
                  "octex: expected a tensor in device memory");
  else
    OCTEX_EXPECTS(dev == kDLCPU || dev == kDLCUDAHost || dev == kDLCUDAManaged,
                  "octex: expected a tensor in host memory");
  OCTEX_EXPECTS(t.ndim == 2, "octex: the DLPack tensor has the wrong number of dimensions");
  OCTEX_EXPECTS(t.dtype.code == dl_code<T>::value && t.dtype.bits == 8 * sizeof(T) && t.dtype.lanes == 1,
                "octex: the DLPack tensor has the wrong data type");
  if (t.strides != nullptr) {
    int64_t expect = 1;
    for (int i = 1; i >= 0; --i) {
      OCTEX_EXPECTS(t.shape[i] == 1 || t.strides[i] == expect,
                    "octex: the DLPack tensor must be dense and row major");
      expect *= t.shape[i];
    }
  }
  *data = reinterpret_cast<T*>(static_cast<char*>(t.data) + t.byte_offset);
  *rows = t.shape[0];
  *cols = t.shape[1];
}

void load_into(cuvsResources_t res, const char* path, cuvsOctexLoadParams_t params, int rank,
               int world, cuvsOctexIndex_t index)
{
  OCTEX_EXPECTS(index != nullptr, "octex: the index handle is NULL");
  OCTEX_EXPECTS(index->addr == 0, "octex: the index handle already holds an index");
  OCTEX_EXPECTS(path != nullptr, "octex: the index directory is NULL");
  auto p  = params != nullptr ? to_cpp(*params) : octex_b200::load_params{};
  p.rank  = rank;
  p.world = world;
  index->addr = reinterpret_cast<uintptr_t>(
    new octex_b200::index(octex_b200::load(as_res(res), std::string(path), p)));
}

}  // namespace

extern "C" {

// ---- resources and error text ------------------------------------------------------------------

cuvsError_t cuvsResourcesCreate(cuvsResources_t* res)
{
  return translate([=] { *res = reinterpret_cast<cuvsResources_t>(new resources_box{}); });
}

cuvsError_t cuvsResourcesDestroy(cuvsResources_t res)
{
  return translate([=] { delete reinterpret_cast<resources_box*>(res); });
}

cuvsError_t cuvsStreamSet(cuvsResources_t res, void* stream)
{
  return translate([=] {
    OCTEX_EXPECTS(res != 0, "octex: the resources handle is NULL");
    reinterpret_cast<resources_box*>(res)->res.stream = static_cast<cudaStream_t>(stream);
  });
}

cuvsError_t cuvsStreamGet(cuvsResources_t res, void** stream)
{
  return translate([=] { *stream = as_res(res).stream; });
}

cuvsError_t cuvsStreamSync(cuvsResources_t res)
{
  return translate([=] { OCTEX_CUDA_TRY(cudaStreamSynchronize(as_res(res).stream)); });
}

const char* cuvsGetLastErrorText(void) { return g_last_error.empty() ? nullptr : g_last_error.c_str(); }

void cuvsSetLastErrorText(const char* text) { g_last_error = text != nullptr ? text : ""; }

// ---- parameter structs (defaults of the C++ API) ------------------------------------------------

cuvsError_t cuvsOctexIndexParamsCreate(cuvsOctexIndexParams_t* params)
{
  return translate([=] {
    auto* p = new cuvsOctexIndexParams{};
    p->copies = 200, p->blocks = 4, p->pca_dims = 64;
    p->spacings = nullptr, p->n_spacings = 0;
    p->list_len = 64, p->min_cell = 1, p->log_buckets = 20, p->sketch_width = 0, p->table_len = 64;
    p->reverse_edges = true, p->exact_lists = false, p->list_probes = 16, p->member_lists = false;
    p->exact_table_max = 20000000, p->table_passes = 3;
    p->table_sketch_order = false, p->write_behind = false, p->seed = 0;
    p->devices = nullptr, p->n_devices = 0;
    *params = p;
  });
}

cuvsError_t cuvsOctexIndexParamsDestroy(cuvsOctexIndexParams_t params)
{
  return translate([=] { delete params; });
}

cuvsError_t cuvsOctexLoadParamsCreate(cuvsOctexLoadParams_t* params)
{
  return translate([=] {
    auto* p = new cuvsOctexLoadParams{};
    p->devices = nullptr, p->n_devices = 0;
    p->placement = OCTEX_PLACEMENT_SHARD;
    p->vectors_on_host = false, p->shard_vectors = false, p->table_on_host = false;
    p->sketch = OCTEX_SKETCH_REPLICATE;
    p->parts = 0, p->copies_per_part = 0, p->copies_limit = 0, p->list_limit = 0;
    *params = p;
  });
}

cuvsError_t cuvsOctexLoadParamsDestroy(cuvsOctexLoadParams_t params)
{
  return translate([=] { delete params; });
}

cuvsError_t cuvsOctexSearchParamsCreate(cuvsOctexSearchParams_t* params)
{
  return translate([=] {
    const octex_b200::search_params d;
    auto* p = new cuvsOctexSearchParams{};
    p->read = d.read, p->starts = d.starts, p->waves = d.waves, p->rerank = d.rerank;
    p->wave_rerank = d.wave_rerank, p->batch = d.batch, p->sketch_rank = d.sketch_rank;
    p->final_rerank = d.final_rerank, p->balanced_gather = d.balanced_gather;
    p->fused_merge = d.fused_merge, p->use_graph = d.use_graph;
    *params = p;
  });
}

cuvsError_t cuvsOctexSearchParamsDestroy(cuvsOctexSearchParams_t params)
{
  return translate([=] { delete params; });
}

// ---- index handle -------------------------------------------------------------------------------

cuvsError_t cuvsOctexIndexCreate(cuvsOctexIndex_t* index)
{
  return translate([=] { *index = new cuvsOctexIndex{0}; });
}

cuvsError_t cuvsOctexIndexDestroy(cuvsOctexIndex_t index)
{
  return translate([=] {
    if (index == nullptr) return;
    if (index->addr != 0) delete reinterpret_cast<octex_b200::index*>(index->addr);
    delete index;
  });
}

cuvsError_t cuvsOctexIndexGetSize(cuvsOctexIndex_t index, int64_t* size)
{
  return translate([=] { *size = as_index(*index)->size(); });
}

cuvsError_t cuvsOctexIndexGetDim(cuvsOctexIndex_t index, int64_t* dim)
{
  return translate([=] { *dim = as_index(*index)->dim(); });
}

cuvsError_t cuvsOctexIndexGetCopies(cuvsOctexIndex_t index, int32_t* copies)
{
  return translate([=] { *copies = as_index(*index)->copies(); });
}

cuvsError_t cuvsOctexIndexGetNumDevices(cuvsOctexIndex_t index, int32_t* n_devices)
{
  return translate([=] { *n_devices = static_cast<int32_t>(as_index(*index)->devices().size()); });
}

cuvsError_t cuvsOctexIndexGetDevices(cuvsOctexIndex_t index, int32_t* devices)
{
  return translate([=] {
    auto const& d = as_index(*index)->devices();
    for (size_t i = 0; i < d.size(); ++i)
      devices[i] = d[i];
  });
}

cuvsError_t cuvsOctexIndexGetDeviceBytes(cuvsOctexIndex_t index, int64_t* bytes)
{
  return translate([=] {
    const auto b = as_index(*index)->device_bytes();
    for (size_t i = 0; i < b.size(); ++i)
      bytes[i] = b[i];
  });
}

// ---- build, load, search ------------------------------------------------------------------------

cuvsError_t cuvsOctexBuild(cuvsResources_t res, cuvsOctexIndexParams_t params,
                           DLManagedTensor* dataset, const char* path)
{
  return translate([=] {
    OCTEX_EXPECTS(path != nullptr, "octex: the index directory is NULL");
    OCTEX_EXPECTS(params != nullptr && dataset != nullptr, "octex: a build argument is NULL");
    DLTensor const& t = dataset->dl_tensor;
    OCTEX_EXPECTS(t.dtype.code == kDLFloat && (t.dtype.bits == 32 || t.dtype.bits == 16) && t.dtype.lanes == 1,
                  "octex: the dataset must be float32 or float16");
    OCTEX_EXPECTS(t.ndim == 2, "octex: the DLPack tensor has the wrong number of dimensions");
    if (t.strides != nullptr)
      OCTEX_EXPECTS((t.shape[1] == 1 || t.strides[1] == 1) && (t.shape[0] == 1 || t.strides[0] == t.shape[1]),
                    "octex: the DLPack tensor must be dense and row major");
    octex_b200::index_params p;
    p.copies = params->copies, p.blocks = params->blocks, p.pca_dims = params->pca_dims;
    if (params->spacings != nullptr && params->n_spacings > 0)
      p.spacings.assign(params->spacings, params->spacings + params->n_spacings);
    p.list_len = params->list_len, p.min_cell = params->min_cell, p.log_buckets = params->log_buckets;
    p.sketch_width = params->sketch_width, p.table_len = params->table_len;
    p.reverse_edges = params->reverse_edges, p.seed = params->seed;
    p.exact_lists = params->exact_lists, p.list_probes = params->list_probes, p.member_lists = params->member_lists;
    p.exact_table_max = params->exact_table_max, p.table_passes = params->table_passes;
    p.table_sketch_order = params->table_sketch_order, p.write_behind = params->write_behind;
    if (params->devices != nullptr && params->n_devices > 0)
      p.devices.assign(params->devices, params->devices + params->n_devices);
    OCTEX_EXPECTS(p.devices.size() <= 1, "octex: this builder works on one GPU (index_params::devices names several)");
    int cur = 0;
    OCTEX_CUDA_TRY(cudaGetDevice(&cur));
    if (!p.devices.empty()) OCTEX_CUDA_TRY(cudaSetDevice(p.devices[0]));
    octex_b200::build_dataset d;
    d.data = static_cast<const char*>(t.data) + t.byte_offset;
    d.f16  = t.dtype.bits == 16;
    d.rows = t.shape[0], d.dim = t.shape[1];
    try {
      octex_b200::build(as_res(res), p, d, std::string(path));
    } catch (...) {
      cudaSetDevice(cur);
      throw;
    }
    OCTEX_CUDA_TRY(cudaSetDevice(cur));
  });
}

cuvsError_t octexB200Build(cuvsResources_t res, cuvsOctexIndexParams_t params, const void* dataset,
                           int64_t rows, int64_t dim, int32_t f16, int32_t verbose, const char* path)
{
  return translate([=] {
    OCTEX_EXPECTS(path != nullptr && params != nullptr && dataset != nullptr, "octex: a build argument is NULL");
    octex_b200::index_params p;
    p.copies = params->copies, p.blocks = params->blocks, p.pca_dims = params->pca_dims;
    if (params->spacings != nullptr && params->n_spacings > 0)
      p.spacings.assign(params->spacings, params->spacings + params->n_spacings);
    p.list_len = params->list_len, p.min_cell = params->min_cell, p.log_buckets = params->log_buckets;
    p.sketch_width = params->sketch_width, p.table_len = params->table_len;
    p.reverse_edges = params->reverse_edges, p.seed = params->seed;
    p.exact_table_max = params->exact_table_max, p.table_passes = params->table_passes;
    p.table_sketch_order = params->table_sketch_order;
    p.verbose = verbose != 0;
    octex_b200::build_dataset d;
    d.data = dataset, d.f16 = f16 != 0, d.rows = rows, d.dim = dim;
    octex_b200::build(as_res(res), p, d, std::string(path));
  });
}

cuvsError_t octexB200ExactNeighbors(cuvsResources_t res, const void* rows_f16, int64_t n, int32_t dim, int32_t k,
                                    int32_t method, int32_t* ids, float* distances)
{
  return translate([=] {
    OCTEX_EXPECTS(rows_f16 != nullptr && ids != nullptr && distances != nullptr, "octex: an argument is NULL");
    octex_b200::exact_neighbors(static_cast<const __half*>(rows_f16), n, dim, k, method, ids, distances,
                                as_res(res).stream);
  });
}

cuvsError_t cuvsOctexLoad(cuvsResources_t res, const char* path, cuvsOctexLoadParams_t params,
                          cuvsOctexIndex_t index)
{
  return translate([=] { load_into(res, path, params, 0, 1, index); });
}

cuvsError_t octexB200LoadRank(cuvsResources_t res, const char* path, cuvsOctexLoadParams_t params,
                              int32_t rank, int32_t world, cuvsOctexIndex_t index)
{
  return translate([=] { load_into(res, path, params, rank, world, index); });
}

cuvsError_t octexB200Attach(cuvsResources_t res, const octexB200Arrays* a,
                            cuvsOctexLoadParams_t params, int32_t rank, int32_t world,
                            cuvsOctexIndex_t index)
{
  return translate([=] {
    OCTEX_EXPECTS(index != nullptr && a != nullptr, "octex: an attach argument is NULL");
    OCTEX_EXPECTS(index->addr == 0, "octex: the index handle already holds an index");
    auto p  = params != nullptr ? to_cpp(*params) : octex_b200::load_params{};
    p.rank  = rank;
    p.world = world;
    octex_b200::index_arrays x;
    x.n = a->n, x.dim = a->dim, x.copies = a->copies, x.blocks = a->blocks;
    x.list_len = a->list_len, x.log_buckets = a->log_buckets, x.sketch_width = a->sketch_width;
    x.table_len = a->table_len;
    if (a->spacings != nullptr && a->n_spacings > 0)
      x.spacings.assign(a->spacings, a->spacings + a->n_spacings);
    else
      x.spacings = {2.0f, 2.5f, 3.2f, 4.0f, 5.0f};
    x.stride = a->stride, x.mmax = a->mmax;
    x.mean = a->mean, x.proj = a->proj, x.shift = a->shift, x.lists = a->lists, x.keys = a->keys;
    x.offsets = a->offsets, x.base = a->base, x.basis = a->sketch_basis, x.scale = a->sketch_scale;
    x.sketch = a->sketch, x.vectors = a->vectors, x.table = a->table;
    x.borrow = a->borrow != 0;
    index->addr = reinterpret_cast<uintptr_t>(
      new octex_b200::index(octex_b200::attach(as_res(res), x, p)));
  });
}

cuvsError_t cuvsOctexSearch(cuvsResources_t res, cuvsOctexSearchParams_t params,
                            cuvsOctexIndex_t index, DLManagedTensor* queries,
                            DLManagedTensor* neighbors, DLManagedTensor* distances)
{
  return translate([=] {
    OCTEX_EXPECTS(params != nullptr && index != nullptr && queries != nullptr,
                  "octex: a search argument is NULL");
    const auto p   = to_cpp(*params);
    auto const& ix = *as_index(*index);
    const auto t   = queries->dl_tensor.device.device_type;
    const bool dev = t == kDLCUDA || t == kDLCUDAManaged;
    float* q       = nullptr;
    int64_t* nb    = nullptr;
    float* ds      = nullptr;
    int64_t qr = 0, qc = 0, nr = 0, nc = 0, dr = 0, dc = 0;
    matrix_of<float>(queries, dev, &q, &qr, &qc);
    matrix_of<int64_t>(neighbors, dev, &nb, &nr, &nc);
    matrix_of<float>(distances, dev, &ds, &dr, &dc);
    if (dev)
      octex_b200::search(as_res(res), p, ix, octex_b200::device_matrix_view<const float>{q, qr, qc},
                         octex_b200::device_matrix_view<int64_t>{nb, nr, nc},
                         octex_b200::device_matrix_view<float>{ds, dr, dc});
    else
      octex_b200::search(as_res(res), p, ix, octex_b200::host_matrix_view<const float>{q, qr, qc},
                         octex_b200::host_matrix_view<int64_t>{nb, nr, nc},
                         octex_b200::host_matrix_view<float>{ds, dr, dc});
  });
}

cuvsError_t octexB200Search(cuvsResources_t res, cuvsOctexSearchParams_t params,
                            cuvsOctexIndex_t index, const float* queries, int64_t n_queries,
                            int64_t dim, int64_t* neighbors, float* distances, int64_t k,
                            int32_t on_device)
{
  return translate([=] {
    OCTEX_EXPECTS(params != nullptr && index != nullptr, "octex: a search argument is NULL");
    OCTEX_EXPECTS(n_queries == 0 || (queries != nullptr && neighbors != nullptr && distances != nullptr),
                  "octex: a search array is NULL");
    octex_b200::detail::search_impl(as_res(res), to_cpp(*params), *as_index(*index), queries,
                                    n_queries, dim, neighbors, distances, k, on_device == 0, false);
  });
}

cuvsError_t octexB200SearchResident(cuvsResources_t res, cuvsOctexSearchParams_t params,
                                    cuvsOctexIndex_t index, int64_t n_queries, int64_t k)
{
  return translate([=] {
    OCTEX_EXPECTS(params != nullptr && index != nullptr, "octex: a search argument is NULL");
    auto const& ix = *as_index(*index);
    const auto p   = to_cpp(*params);
    OCTEX_EXPECTS(n_queries <= std::max(p.batch, 1),
                  "octex: resident search needs the whole query set in one batch");
    octex_b200::detail::search_impl(as_res(res), p, ix, nullptr, n_queries, ix.dim(), nullptr,
                                    nullptr, k, false, true);
    OCTEX_CUDA_TRY(cudaStreamSynchronize(ix.impl().part.stream));
    check_last(ix.impl());
  });
}

cuvsError_t octexB200CheckLast(cuvsOctexIndex_t index)
{
  return translate([=] {
    auto& ix = as_index(*index)->impl();
    OCTEX_CUDA_TRY(cudaStreamSynchronize(ix.part.stream));
    check_last(ix);
  });
}

cuvsError_t octexB200SetTable(cuvsOctexIndex_t index, const int32_t* table, int32_t table_len)
{
  return translate([=] { octex_b200::detail::set_table(as_index(*index)->impl(), table, table_len); });
}

cuvsError_t octexB200SearchedTable(cuvsResources_t res, cuvsOctexIndex_t index, int32_t table_len, int32_t passes,
                                   int32_t reverse_edges, int32_t sketch_order, int32_t* table)
{
  return translate([=] {
    octex_b200::searched_table(as_res(res), *as_index(*index), table_len, passes, reverse_edges != 0,
                               sketch_order != 0, table, false);
  });
}

cuvsError_t octexB200MemoryReport(cuvsOctexIndex_t index, int64_t* bytes)
{
  return translate([=] {
    OCTEX_EXPECTS(bytes != nullptr, "octex: a NULL report");
    auto& ix = as_index(*index)->impl();
    auto const& p = ix.part;
    auto dev = [](octex_b200::dbuf const& b) { return b.host ? int64_t{0} : static_cast<int64_t>(b.size); };
    bytes[0] = p.device;
    bytes[1] = dev(p.lists) + dev(p.base) + dev(p.cell_table) + dev(p.cell_off) + dev(p.cell_mask) + dev(p.level_on);
    bytes[2] = dev(p.sketch) + dev(p.sketch_norm);
    bytes[3] = dev(p.table);
    bytes[4] = dev(p.vectors);
    bytes[5] = dev(p.ut) + dev(p.shift) + dev(p.inv_f) + dev(p.mean) + dev(p.basis) + dev(p.scale) +
               dev(p.table_rows.ptrs) + dev(p.sketch_rows.ptrs) + dev(p.vector_rows.ptrs);
    bytes[6] = 0;
    std::lock_guard<std::mutex> lock(ix.mu);
    for (auto const& kv : ix.plans)
      bytes[6] += kv.second->buffer_bytes;
  });
}

cuvsError_t octexB200ProfileBatch(cuvsResources_t res, cuvsOctexSearchParams_t params,
                                  cuvsOctexIndex_t index, int64_t n_queries, int64_t k, float* ms,
                                  int32_t capacity, int32_t* count)
{
  return translate([=] {
    OCTEX_EXPECTS(params != nullptr && index != nullptr && count != nullptr,
                  "octex: a profile argument is NULL");
    auto t = octex_b200::detail::profile_batch(as_res(res), to_cpp(*params), *as_index(*index),
                                               n_queries, k);
    *count = static_cast<int32_t>(t.size());
    for (int i = 0; i < *count && i < capacity && ms != nullptr; i++)
      ms[i] = t[i];
  });
}

// ---- observation --------------------------------------------------------------------------------

cuvsError_t octexB200SetDebug(cuvsOctexIndex_t index, int32_t stats, int32_t taps)
{
  return translate([=] {
    auto& ix = as_index(*index)->impl();
    std::lock_guard<std::mutex> lock(ix.mu);
    ix.debug.stats = stats != 0;
    ix.debug.taps  = taps != 0;
  });
}

cuvsError_t octexB200CommUniqueId(void* id128)
{
  return translate([=] {
    OCTEX_EXPECTS(id128 != nullptr, "octex: a NULL id buffer");
    octex_b200::detail::communicator::unique_id(id128);
  });
}

cuvsError_t octexB200CommInit(cuvsOctexIndex_t index, const void* id128)
{
  return translate([=] {
    OCTEX_EXPECTS(id128 != nullptr, "octex: a NULL id buffer");
    auto& ix = as_index(*index)->impl();
    OCTEX_EXPECTS(ix.world > 1, "octex: the index belongs to a single process");
    {
      std::lock_guard<std::mutex> lock(ix.mu);
      ix.plans.clear();
      ix.comm = std::make_unique<octex_b200::detail::communicator>(id128, ix.rank, ix.world,
                                                                   ix.part.device);
    }
    octex_b200::detail::connect_rows(ix);  // arrays dealt by rows: map the other processes' ranges
  });
}

cuvsError_t octexB200CommDisconnect(cuvsOctexIndex_t index)
{
  return translate([=] {
    auto& ix = as_index(*index)->impl();
    octex_b200::detail::disconnect_rows(ix);
  });
}

cuvsError_t octexB200SetProjection(cuvsOctexIndex_t index, int32_t ordered)
{
  return translate([=] {
    auto& ix = as_index(*index)->impl();
    std::lock_guard<std::mutex> lock(ix.mu);
    ix.debug.ordered_projection = ordered != 0;
  });
}

cuvsError_t octexB200Fetch(cuvsOctexIndex_t index, const char* name, void* dst, int64_t capacity,
                           int64_t* bytes)
{
  return translate([=] {
    auto& ix = as_index(*index)->impl();
    std::shared_ptr<octex_b200::detail::plan> pl;
    {
      std::lock_guard<std::mutex> lock(ix.mu);
      OCTEX_EXPECTS(!ix.plans.empty(), "octex: nothing to fetch before the first search");
      pl = ix.plans.begin()->second;
    }
    const std::string n(name != nullptr ? name : "");
    octex_b200::dbuf const* b = nullptr;
    if (n == "y") b = &pl->Y;
    else if (n == "qs") b = &pl->qs;
    else if (n == "codes") b = &pl->codes;
    else if (n == "seg") b = &pl->seg;
    else if (n == "cand1") b = &pl->tap_cand;
    else if (n == "cand1_dist") b = &pl->tap_dist;
    else if (n == "n1") b = &pl->tap_n;
    else if (n == "kept1_ids") b = &pl->kept1_i;
    else if (n == "kept1_dist") b = &pl->kept1_d;
    else if (n == "kept_ids") b = &pl->si;
    else if (n == "kept_dist") b = &pl->sd;
    else if (n == "stats") b = &pl->stats;
    else if (n == "phase_lists") b = &pl->phase1;
    else if (n == "phase_rows") b = &pl->phase2;
    OCTEX_EXPECTS(b != nullptr, "octex: unknown array name \"" + n + "\"");
    OCTEX_EXPECTS(b->ptr != nullptr, "octex: \"" + n + "\" is not kept (see octexB200SetDebug)");
    if (bytes != nullptr) *bytes = static_cast<int64_t>(b->size);
    if (dst == nullptr) return;
    OCTEX_EXPECTS(capacity >= static_cast<int64_t>(b->size), "octex: the destination is too small");
    std::lock_guard<std::mutex> lock(pl->mu);
    OCTEX_CUDA_TRY(cudaSetDevice(pl->device));
    OCTEX_CUDA_TRY(cudaStreamSynchronize(ix.part.stream));
    OCTEX_CUDA_TRY(cudaMemcpy(dst, b->ptr, b->size, cudaMemcpyDeviceToHost));
  });
}

cuvsError_t octexB200CellCodes(const float* y, int64_t n, int32_t blocks, float inv_f, int64_t* codes)
{
  return translate([=] {
    OCTEX_EXPECTS((blocks >= 1 && blocks <= 6) || blocks == 8, "octex: blocks must be 1-6 or 8");
    OCTEX_EXPECTS(n >= 0 && (n == 0 || (y != nullptr && codes != nullptr)), "octex: a NULL array");
    if (n == 0) return;
    int dev = 0;
    OCTEX_CUDA_TRY(cudaGetDevice(&dev));
    octex_b200::dbuf dy(dev, static_cast<size_t>(n) * 8 * blocks * sizeof(float));
    octex_b200::dbuf dc(dev, static_cast<size_t>(n) * sizeof(int64_t));
    OCTEX_CUDA_TRY(cudaMemcpy(dy.ptr, y, dy.size, cudaMemcpyHostToDevice));
    octex_b200::kernels::cell_codes_f32(dy.as<float>(), n, blocks, inv_f, dc.as<long long>(), nullptr);
    OCTEX_CUDA_TRY(cudaGetLastError());
    OCTEX_CUDA_TRY(cudaDeviceSynchronize());
    OCTEX_CUDA_TRY(cudaMemcpy(codes, dc.ptr, dc.size, cudaMemcpyDeviceToHost));
  });
}

}  // extern "C"
