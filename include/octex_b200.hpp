// C++ interface of the B200 search library: the search-side surface of
// cuvs::neighbors::octex (hpdic/octex, cpp/include/cuvs/neighbors/octex.hpp), without the RAFT
// types. Names, defaults and meaning of every parameter are those of the reference; what stands in
// for a RAFT type says so.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace octex_b200 {

/// Stand-in for raft::resources: the search uses nothing of it but the CUDA stream
/// (cpp/src/neighbors/octex/search.cu:835); load ignores it (load.cu:208).
struct resources {
  cudaStream_t stream = nullptr;
};

/// Stand-ins for raft::host_matrix_view / raft::device_matrix_view<T, int64_t, row_major>: the
/// reference reads only data_handle() and extent(i) of them (search.cu:1027-1063).
template <typename T>
struct host_matrix_view {
  T* data      = nullptr;
  int64_t rows = 0, cols = 0;
};
template <typename T>
struct device_matrix_view {
  T* data      = nullptr;
  int64_t rows = 0, cols = 0;
};

/// octex.hpp:101-135
struct search_params {
  int read             = 32;    ///< list entries read per copy in the first round
  int starts           = 128;   ///< best first-round hits kept as start points of the waves
  int waves            = 2;     ///< secondary waves over the neighbor table (0: first round only)
  int rerank           = 128;   ///< exact rerank depth of the first round
  int wave_rerank      = 128;   ///< exact rerank depth of every wave
  int batch            = 10000; ///< queries per captured batch
  bool sketch_rank     = false; ///< rank by the sketch, rerank exactly only at the end
  int final_rerank     = 32;    ///< sketch-rank mode: kept entries reranked exactly at the end
  /// Ablation switches of the reference. This library has one implementation of the gather and of
  /// the merge; those two fields are accepted and ignored.
  bool balanced_gather = true;
  bool fused_merge     = true;
  /// false: direct kernel launches for every batch instead of replaying its CUDA graph.
  bool use_graph       = true;
};

/// octex.hpp:32-92. The builder of this library makes member lists (the rows of a cell nearest its
/// centre first, the reference's member_lists mode) and a neighbor table that is exact up to
/// exact_table_max rows and made by the index's own search in table_passes passes above that
/// (table_sketch_order: without the exact rerank of those searches); the fields that choose among
/// the reference's other build strategies (exact_lists, list_probes, member_lists, write_behind,
/// devices) are accepted and have no effect.
struct index_params {
  int copies       = 200;   ///< random projections of the dataset
  int blocks       = 4;     ///< E8 blocks per copy (8 coordinates each)
  int pca_dims     = 64;    ///< principal directions a copy's projection is drawn from
  std::vector<float> spacings{};  ///< lattice spacings, fine to coarse (empty: 2, 2.5, 3.2, 4, 5)
  int list_len     = 64;    ///< rows listed per cell
  int min_cell     = 1;     ///< cells with fewer rows are dropped (not at the coarsest spacing)
  int log_buckets  = 20;    ///< log2 of the buckets the cells of a (copy, spacing) are hashed into
  int sketch_width = 0;     ///< int8 sketch coordinates (0: chosen from the dimension)
  int table_len    = 64;    ///< neighbors per row of the neighbor table (0: none)
  bool reverse_edges = true;  ///< merge reverse edges into the table (half rule)
  bool exact_lists = false, member_lists = false, table_sketch_order = false, write_behind = false;
  int list_probes = 16, table_passes = 3;
  int64_t exact_table_max = 20000000;
  uint64_t seed = 0;
  std::vector<int> devices{};
  bool verbose = false;  ///< progress lines on stderr (the reference's OCTEX_VERBOSE)
};

/// The dataset of a build: n rows of dim float32 or float16 values, row major, in host or device
/// memory (the two build overloads of octex.hpp:214-222 in one struct).
struct build_dataset {
  const void* data = nullptr;
  bool f16         = false;
  int64_t rows = 0, dim = 0;
};

/// Build an index of the dataset into the directory `path` (octex.hpp:214-222), on the current
/// GPU. The directory is complete once its meta.json exists.
void build(resources const& res, index_params const& params, build_dataset const& dataset,
           std::string const& path);

/// The sketch width the builder chooses for a dimension when index_params::sketch_width is 0.
auto auto_sketch_width(int64_t dim) -> int;

/// octex.hpp:138-143
enum class placement : int { replicate = 0, shard = 1 };
/// octex.hpp:146-153
enum class sketch_placement : int { replicate = 0, shard = 1, host = 2 };

/// octex.hpp:155-176, plus the rank of this process among the processes that hold the index.
struct load_params {
  std::vector<int> devices{};  ///< GPU of this process (empty: the current device)
  placement mode       = placement::shard;
  bool vectors_on_host = false;
  bool shard_vectors   = false;
  bool table_on_host   = false;
  sketch_placement sketch = sketch_placement::replicate;
  int parts            = 0;
  int copies_per_part  = 0;
  int copies_limit     = 0;
  int list_limit       = 0;
  /// One process per GPU: this process is `rank` of `world` processes sharing the index. With
  /// shard placement it holds copies [C*rank/world, C*(rank+1)/world); with replicate, all.
  int rank  = 0;
  int world = 1;
};

/// Arrays of an index handed over in memory instead of through a directory: the same arrays, with
/// the same dtypes and shapes, that the directory holds (docs/design.md:27-48). Pointers may be host
/// or device memory. With `borrow` set, device arrays that need no re-layout (lists, keys, offsets,
/// sketch, vectors, table) are used in place and must outlive the index.
struct index_arrays {
  int64_t n = 0, dim = 0;
  int copies = 0, blocks = 4, list_len = 0, log_buckets = 20, sketch_width = 0, table_len = 0;
  std::vector<float> spacings;
  int64_t stride = 0;  ///< entries per copy in lists
  int64_t mmax   = 0;  ///< keys per (copy, level)
  const float* mean = nullptr;       ///< [dim]
  const float* proj = nullptr;       ///< [copies, dim, 8*blocks]
  const float* shift = nullptr;      ///< [copies, 8*blocks]
  const int32_t* lists = nullptr;    ///< [copies, stride]
  const int64_t* keys = nullptr;     ///< [copies, levels, mmax]
  const int32_t* offsets = nullptr;  ///< [copies, levels, 2^log_buckets + 1]
  const int32_t* base = nullptr;     ///< [copies, levels]
  const int64_t* cells = nullptr;    ///< [copies, levels] (may be null)
  const float* basis = nullptr;      ///< [dim, sketch_width]
  const float* scale = nullptr;      ///< [sketch_width]
  const int8_t* sketch = nullptr;    ///< [n, sketch_width]
  const void* vectors = nullptr;     ///< [n, dim] fp16
  const int32_t* table = nullptr;    ///< [n, table_len] (null when table_len == 0)
  bool borrow = false;
};

namespace detail {
struct index_impl;
}

/// An index placed on the GPU of this process (octex.hpp:187-204).
class index {
 public:
  explicit index(std::shared_ptr<detail::index_impl> impl);
  index(index&&) noexcept;
  auto operator=(index&&) noexcept -> index&;
  ~index();
  [[nodiscard]] auto size() const noexcept -> int64_t;
  [[nodiscard]] auto dim() const noexcept -> int64_t;
  [[nodiscard]] auto copies() const noexcept -> int;
  [[nodiscard]] auto devices() const noexcept -> std::vector<int> const&;
  [[nodiscard]] auto device_bytes() const -> std::vector<int64_t>;
  [[nodiscard]] auto impl() const noexcept -> detail::index_impl&;

 private:
  std::shared_ptr<detail::index_impl> impl_;
};

/// Load an index directory onto the GPU (octex.hpp:225-226).
auto load(resources const& res, std::string const& path, load_params const& params = {}) -> index;

/// Place an index from arrays in memory (no counterpart in the reference, which always goes
/// through a directory; same placement rules as load).
auto attach(resources const& res, index_arrays const& arrays, load_params const& params = {}) -> index;

/// k nearest neighbors of every query, k = neighbors.cols (octex.hpp:241-253). Host results are
/// complete on return; device results are ordered on res.stream.
void search(resources const& res, search_params const& params, index const& idx,
            host_matrix_view<const float> queries, host_matrix_view<int64_t> neighbors,
            host_matrix_view<float> distances);
void search(resources const& res, search_params const& params, index const& idx,
            device_matrix_view<const float> queries, device_matrix_view<int64_t> neighbors,
            device_matrix_view<float> distances);

}  // namespace octex_b200
