// The index as the search kernels read it: arrays of one process's GPU and their layout.
//
// Layout (the reference's is in cpp/src/neighbors/octex/detail/index_impl.hpp:115-177 of
// hpdic/octex; differences are marked *):
//   lists   i32 [Cg, stride]     cell rows of list_len ids, nearest to the cell centre first
// * cell_table {i64 key, i32 row, pad} [sum of the (copy, level) table sizes]: the cells of every
//                                (copy, level) in an open-addressing table at most half full (slot =
//                                low bits of the code, linear probing), with cell_off i64 [Cg, L]
//                                (first slot) and cell_mask i32 [Cg, L] (slots - 1). Built at placement
//                                from the directory's keys i64 [C, L, mmax] and the cell counts in its
//                                offsets i32 [C, L, T + 1]; the reference keeps those two arrays on the
//                                GPU and walks a bucket of keys per lookup
//   base    i32 [Cg, L]          first list row of a level inside the copy
// * ut      f16 [Cg * 8b, ldu]   projections, one row per projected coordinate, K-major
//                                (ldu = dim rounded up to 64, zero padded): the operand layout of
//                                the tensor-core projection (the reference keeps [dim, Cg * 8b])
//   shift   f16 [Cg * 8b]        inv_f f32 [L]     mean f32 [dim]
//   basis   f32 [dim, S]         scale f32 [S]     sketch i8 [n, S]
//   vectors f16 [n, dim]         table i32 [n, table_len]
// * level_on u8 [Cg, L]          1 when the level of the copy holds at least one cell
// * sketch_norm f32 [n]          sum_k (code_k scale_k)^2 of every sketch row, computed at placement
//                                (the row's constant in the integer form of the sketch distance)
#pragma once

#include "comm.hpp"
#include "common.hpp"

#include <octex_b200.hpp>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace octex_b200::detail {

struct plan;

/// Observation switches of an index (off in normal use; tests and the benchmark's byte
/// accounting turn them on). Changing them rebuilds the plan.
struct debug_options {
  bool stats = false;  ///< per-query counters of what the kernels read
  bool taps  = false;  ///< keep the intermediate arrays of the last batch for inspection
  /// Project with the kernel that sums in dimension order (bit-comparable with the CPU checker)
  /// instead of the tensor-core kernel.
  bool ordered_projection = false;
};

/// An array whose rows are dealt over the processes in ranges of rows_per (load.cu:315,406-427 of
/// the reference): this process holds rows [row0, row0 + own rows) in `mine`; after the processes
/// are connected, `ptrs` (device, one pointer per process) gives every range's address, the other
/// processes' memory being mapped into this one.
struct dealt_rows {
  bool on          = false;
  int64_t rows_per = 0, row0 = 0;
  dbuf ptrs;                  // long long [world], null until connected
  std::vector<void*> opened;  // mappings of other processes' memory, closed with the index
};

struct device_part {
  int device     = 0;
  int copies     = 0;  // copies held by this process
  int copy0      = 0;  // first of them
  int64_t stride = 0;
  int64_t mmax   = 0;
  int ldu        = 0;
  dbuf lists, base, ut, shift, inv_f, mean, basis, scale, sketch, vectors, table, level_on;
  dbuf cell_table, cell_off, cell_mask;  // open-addressing table of the cells of every (copy, level)
  dbuf sketch_norm;                      // f32 [n]: sum_k (code_k scale_k)^2 of every sketch row
  dealt_rows table_rows, sketch_rows, vector_rows;
  cudaStream_t stream = nullptr;
  cudaStream_t second = nullptr;  // created when a search first alternates its batches between two streams
  int64_t bytes       = 0;

  device_part() = default;
  device_part(device_part const&) = delete;
  ~device_part()
  {
    int cur = 0;
    cudaGetDevice(&cur);
    cudaSetDevice(device);
    // mappings still open here were not released by disconnect_rows (the collective way out):
    // closing them is all a single process can do
    for (dealt_rows* d : {&table_rows, &sketch_rows, &vector_rows})
      for (void* p : d->opened)
        cudaIpcCloseMemHandle(p);
    if (stream != nullptr) cudaStreamDestroy(stream);
    if (second != nullptr) cudaStreamDestroy(second);
    cudaSetDevice(cur);
  }
};

struct index_impl {
  std::string path;
  load_params params;
  int64_t n = 0, dim = 0;
  int copies = 0;  // copies loaded over all processes
  int blocks = 4, list_len = 0, log_buckets = 20, sketch_width = 0, table_len = 0;
  std::vector<float> spacings;
  std::vector<int> devices;
  int rank = 0, world = 1;
  device_part part;
  std::mutex mu;  // guards plans
  std::map<std::string, std::shared_ptr<plan>> plans;
  debug_options debug;
  std::unique_ptr<communicator> comm;  // set when world > 1 (octexB200CommInit)
  ~index_impl();
};

/// Host-side view of the arrays of an index (directory or memory) that placement reads from.
struct source_arrays {
  index_arrays a;
  int all_copies = 0;
};

void place(index_impl& ix, source_arrays const& src);
/// After the communicator exists: exchange the addresses of the row ranges dealt over the
/// processes (a collective: every process calls it).
void connect_rows(index_impl& ix);
/// The way back, also a collective: every process drops its plans, waits for its own stream,
/// unmaps the other processes' ranges, and only after all of them have done so (a barrier on the
/// communicator) does any of them go on to free the range it exported; the communicator goes last.
/// Without it a process that closes early would free memory another still has mapped.
void disconnect_rows(index_impl& ix);

/// Replace the neighbor table of an index held by one process (load.cu:498-564 of the reference:
/// set_table / drop_table): table int32 [n, table_len] in host or device memory is copied to the
/// GPU of the index; table_len 0 (table may be null) drops the table. Plans made before are dropped.
void set_table(index_impl& ix, const int32_t* table, int table_len);

}  // namespace octex_b200::detail
