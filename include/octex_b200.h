/* C interface of the B200 search library.
 *
 * The cuvsOctex* functions, structs and enums below are the ones a program written against the
 * reference's C API binds (hpdic/octex, c/include/cuvs/neighbors/octex.h): same names, field
 * order, defaults, ownership and error conventions. The few cuvs* functions the reference takes
 * from the cuVS C library (resources, stream, last error text) are provided too, so that this one
 * shared library satisfies such a program. The octexB200* functions are the same operations with
 * plain pointers and sizes, for callers without DLPack (ctypes, cgo, JNI).
 *
 * Every function returns CUVS_SUCCESS or CUVS_ERROR; after CUVS_ERROR, cuvsGetLastErrorText()
 * returns the message of the failing call on this thread (c/src/core/exceptions.hpp:17-33).
 */
#ifndef OCTEX_B200_H_
#define OCTEX_B200_H_

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OCTEX_B200_EXPORT __attribute__((visibility("default")))

/* ---- what the reference takes from cuVS's C library (cuvs/core/c_api.h) ---- */

typedef enum { CUVS_ERROR = 0, CUVS_SUCCESS = 1 } cuvsError_t;
typedef uintptr_t cuvsResources_t;

OCTEX_B200_EXPORT cuvsError_t cuvsResourcesCreate(cuvsResources_t* res);
OCTEX_B200_EXPORT cuvsError_t cuvsResourcesDestroy(cuvsResources_t res);
/* stream: a cudaStream_t */
OCTEX_B200_EXPORT cuvsError_t cuvsStreamSet(cuvsResources_t res, void* stream);
OCTEX_B200_EXPORT cuvsError_t cuvsStreamGet(cuvsResources_t res, void** stream);
OCTEX_B200_EXPORT cuvsError_t cuvsStreamSync(cuvsResources_t res);
OCTEX_B200_EXPORT const char* cuvsGetLastErrorText(void);
OCTEX_B200_EXPORT void cuvsSetLastErrorText(const char* text);

/* ---- DLPack v1.0 tensor structs, declared here only if dlpack/dlpack.h was not included ---- */
#ifndef DLPACK_DLPACK_H_
#define OCTEX_B200_OWN_DLPACK 1
typedef enum {
  kDLCPU = 1, kDLCUDA = 2, kDLCUDAHost = 3, kDLCUDAManaged = 13
} DLDeviceType;
typedef struct { DLDeviceType device_type; int32_t device_id; } DLDevice;
typedef enum { kDLInt = 0U, kDLUInt = 1U, kDLFloat = 2U } DLDataTypeCode;
typedef struct { uint8_t code; uint8_t bits; uint16_t lanes; } DLDataType;
typedef struct {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides; /* in elements; NULL: compact row-major */
  uint64_t byte_offset;
} DLTensor;
typedef struct DLManagedTensor {
  DLTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(struct DLManagedTensor* self);
} DLManagedTensor;
#endif

/* ---- index build parameters: c/include/cuvs/neighbors/octex.h:31-76 ---- */

struct cuvsOctexIndexParams {
  int32_t copies;
  int32_t blocks;
  int32_t pca_dims;
  const float* spacings;
  int32_t n_spacings;
  int32_t list_len;
  int32_t min_cell;
  int32_t log_buckets;
  int32_t sketch_width;
  int32_t table_len;
  bool reverse_edges;
  bool exact_lists;
  int32_t list_probes;
  bool member_lists;
  int64_t exact_table_max;
  int32_t table_passes;
  bool table_sketch_order;
  bool write_behind;
  uint64_t seed;
  const int32_t* devices;
  int32_t n_devices;
};
typedef struct cuvsOctexIndexParams* cuvsOctexIndexParams_t;
/* octex.h:81-84 */
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexParamsCreate(cuvsOctexIndexParams_t* params);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexParamsDestroy(cuvsOctexIndexParams_t params);

/* ---- load parameters: octex.h:96-140 ---- */

typedef enum { OCTEX_PLACEMENT_REPLICATE = 0, OCTEX_PLACEMENT_SHARD = 1 } cuvsOctexPlacement;
typedef enum {
  OCTEX_SKETCH_REPLICATE = 0, OCTEX_SKETCH_SHARD = 1, OCTEX_SKETCH_HOST = 2
} cuvsOctexSketchPlacement;

struct cuvsOctexLoadParams {
  const int32_t* devices;
  int32_t n_devices;
  cuvsOctexPlacement placement;
  bool vectors_on_host;
  bool shard_vectors;
  bool table_on_host;
  cuvsOctexSketchPlacement sketch;
  int32_t parts;
  int32_t copies_per_part;
  int32_t copies_limit;
  int32_t list_limit;
};
typedef struct cuvsOctexLoadParams* cuvsOctexLoadParams_t;
/* octex.h:146-149 */
OCTEX_B200_EXPORT cuvsError_t cuvsOctexLoadParamsCreate(cuvsOctexLoadParams_t* params);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexLoadParamsDestroy(cuvsOctexLoadParams_t params);

/* ---- search parameters: octex.h:161-184 ---- */

struct cuvsOctexSearchParams {
  int32_t read;
  int32_t starts;
  int32_t waves;
  int32_t rerank;
  int32_t wave_rerank;
  int32_t batch;
  bool sketch_rank;
  int32_t final_rerank;
  bool balanced_gather; /* accepted, ignored: one implementation */
  bool fused_merge;     /* accepted, ignored */
  bool use_graph;       /* false: direct kernel launches instead of replaying the batch graph */
};
typedef struct cuvsOctexSearchParams* cuvsOctexSearchParams_t;
/* octex.h:189-192 */
OCTEX_B200_EXPORT cuvsError_t cuvsOctexSearchParamsCreate(cuvsOctexSearchParams_t* params);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexSearchParamsDestroy(cuvsOctexSearchParams_t params);

/* ---- index handle: octex.h:204-240 ---- */

typedef struct { uintptr_t addr; } cuvsOctexIndex;
typedef cuvsOctexIndex* cuvsOctexIndex_t;

OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexCreate(cuvsOctexIndex_t* index);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexDestroy(cuvsOctexIndex_t index);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexGetSize(cuvsOctexIndex_t index, int64_t* size);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexGetDim(cuvsOctexIndex_t index, int64_t* dim);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexGetCopies(cuvsOctexIndex_t index, int32_t* copies);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexGetNumDevices(cuvsOctexIndex_t index, int32_t* n_devices);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexGetDevices(cuvsOctexIndex_t index, int32_t* devices);
OCTEX_B200_EXPORT cuvsError_t cuvsOctexIndexGetDeviceBytes(cuvsOctexIndex_t index, int64_t* bytes);

/* ---- build, load, search: octex.h:261-295 ---- */

/* The index builder is not part of this library (it covers the search path): returns CUVS_ERROR
 * after the same argument checks as the reference. Directories come from the reference's builder
 * or from the Python tooling of this repository. */
OCTEX_B200_EXPORT cuvsError_t cuvsOctexBuild(cuvsResources_t res, cuvsOctexIndexParams_t params,
                                             DLManagedTensor* dataset, const char* path);
/* cuvsOctexBuild with plain pointers (the shape the Python layer calls): dataset [rows, dim]
 * float32 (f16 = 0) or float16 (f16 = 1), row major, host or device memory; verbose = 1 prints
 * progress on stderr (the reference's OCTEX_VERBOSE, cpp/src/neighbors/octex/detail/build_common.cuh:38-54). */
OCTEX_B200_EXPORT cuvsError_t octexB200Build(cuvsResources_t res, cuvsOctexIndexParams_t params,
                                             const void* dataset, int64_t rows, int64_t dim,
                                             int32_t f16, int32_t verbose, const char* path);

/* Exact k nearest other rows of every row of rows_f16 [n, dim] (fp16, device memory of the current
 * GPU) by squared L2 between the fp16 rows: what the builder's neighbor table starts from (the
 * reference calls cuVS brute force there, cpp/src/neighbors/octex/detail/build_table.cuh:60-142).
 * ids int32 / distances float [n, k] in device memory: nearest first, equal distances by ascending
 * id, -1 / +inf where a row has fewer than k others. method 0: tensor cores when dim is a multiple
 * of 8 and k <= 120, else the plain scan; 1: tensor cores or an error; 2: the plain scan. Returns
 * when the work on the resources' stream is done. */
OCTEX_B200_EXPORT cuvsError_t octexB200ExactNeighbors(cuvsResources_t res, const void* rows_f16, int64_t n,
                                                      int32_t dim, int32_t k, int32_t method, int32_t* ids,
                                                      float* distances);

/* detail::set_table / drop_table of the reference (cpp/src/neighbors/octex/load.cu:498-564): replace
 * the neighbor table of an index held by one process by table int32 [n, table_len] (host or device
 * memory; copied), or drop it (table_len 0, table may be NULL). */
OCTEX_B200_EXPORT cuvsError_t octexB200SetTable(cuvsOctexIndex_t index, const int32_t* table, int32_t table_len);

/* The neighbor table by the index's own search (searched_table of the reference,
 * cpp/src/neighbors/octex/detail/build_table.cuh:648-841): every stored row is searched for
 * 3 table_len / 2 + 1 neighbors in `passes` passes (1 to 3: the first round alone, then 2 and 3 waves
 * over the table of the pass before), ranking by sketch with an exact rerank at the end; the row
 * itself is dropped and, unless reverse_edges is 0, reverse edges are merged in (table_len / 4
 * forward entries first, up to 3 table_len / 4 reverse ones). sketch_order non-zero leaves the
 * answers in sketch order without the exact rerank (table_sketch_order). The index keeps the table of the last
 * pass; table (host memory, int32 [n, table_len], may be NULL) receives it. cuvsOctexBuild takes
 * this way by itself for more rows than exact_table_max. One process, fp16 rows on its GPU. */
OCTEX_B200_EXPORT cuvsError_t octexB200SearchedTable(cuvsResources_t res, cuvsOctexIndex_t index,
                                                     int32_t table_len, int32_t passes, int32_t reverse_edges,
                                                     int32_t sketch_order, int32_t* table);

/* Load an index directory onto the GPU of this process into an empty handle (params NULL: the
 * defaults). octex.h:268-271 */
OCTEX_B200_EXPORT cuvsError_t cuvsOctexLoad(cuvsResources_t res, const char* path,
                                            cuvsOctexLoadParams_t params, cuvsOctexIndex_t index);
/* queries [n, dim] float32, neighbors [n, k] int64, distances [n, k] float32; all on the host or
 * all on a device. Host results are written on return; device results are ordered on the stream
 * of res. octex.h:290-295 */
OCTEX_B200_EXPORT cuvsError_t cuvsOctexSearch(cuvsResources_t res, cuvsOctexSearchParams_t params,
                                              cuvsOctexIndex_t index, DLManagedTensor* queries,
                                              DLManagedTensor* neighbors, DLManagedTensor* distances);

/* ---- the same operations with plain pointers ---- */

/* cuvsOctexSearch (octex.h:290-295) without DLPack. on_device: 0 = the three arrays are host
 * memory, 1 = device memory. */
OCTEX_B200_EXPORT cuvsError_t octexB200Search(cuvsResources_t res, cuvsOctexSearchParams_t params,
                                              cuvsOctexIndex_t index, const float* queries,
                                              int64_t n_queries, int64_t dim, int64_t* neighbors,
                                              float* distances, int64_t k, int32_t on_device);

/* cuvsOctexLoad (octex.h:268-271) for one process per GPU: this process is `rank` of `world`
 * processes that share the index (shard placement deals the copies over the processes as
 * cpp/src/neighbors/octex/load.cu:264-281 deals them over GPUs). */
OCTEX_B200_EXPORT cuvsError_t octexB200LoadRank(cuvsResources_t res, const char* path,
                                                cuvsOctexLoadParams_t params, int32_t rank,
                                                int32_t world, cuvsOctexIndex_t index);

/* Connect the processes that share an index (world > 1). The reference needs no such step: it
 * drives all GPUs from one process and reads across them through peer pointers
 * (cpp/src/neighbors/octex/load.cu:187-202). Here one process calls octexB200CommUniqueId, hands
 * the 128 bytes to the others by any means (a file, MPI, torch.distributed), and every process
 * then calls octexB200CommInit with them; the calls return together. Afterwards every process
 * calls the search with the same queries and parameters and receives all results:
 * replicate placement answers a slice of each batch per process, shard placement runs the first
 * round of all rows over the process's copies, exchanges the kept lists (NCCL send / receive),
 * and runs the waves on the process's slice; an NCCL all-gather brings the slices together.
 * octexB200CommInit is also where arrays dealt by rows (the neighbor table under shard placement,
 * shard_vectors, sketch = SHARD: cpp/src/neighbors/octex/load.cu:315,406-427) become whole: every
 * process publishes a CUDA IPC handle of the row range it holds and maps the others' ranges, which
 * the kernels then read with plain loads. A search before this call fails and says so. */
OCTEX_B200_EXPORT cuvsError_t octexB200CommUniqueId(void* id128);
OCTEX_B200_EXPORT cuvsError_t octexB200CommInit(cuvsOctexIndex_t index, const void* id128);
/* The way out of octexB200CommInit, a COLLECTIVE like it: every process of the index calls it
 * before it destroys its handle. Each process drops its plans, waits for its stream, unmaps the
 * row ranges of the other processes, and returns only after all processes have unmapped (so none
 * frees memory that another still has mapped); the communicator is destroyed. (The reference needs
 * no such call: its one process owns every GPU's memory, cpp/src/neighbors/octex/load.cu:187-202.) */
OCTEX_B200_EXPORT cuvsError_t octexB200CommDisconnect(cuvsOctexIndex_t index);

/* The arrays of an index directory handed over in memory (host or device pointers), with the
 * dtypes and shapes of docs/design.md:27-48. */
typedef struct {
  int64_t n, dim;
  int32_t copies, blocks, list_len, log_buckets, sketch_width, table_len;
  const float* spacings;
  int32_t n_spacings;
  int32_t borrow; /* 1: device arrays needing no re-layout are used in place, not copied */
  int64_t stride; /* entries per copy in lists */
  int64_t mmax;   /* keys per (copy, level) */
  const float* mean;
  const float* proj;
  const float* shift;
  const int32_t* lists;
  const int64_t* keys;
  const int32_t* offsets;
  const int32_t* base;
  const float* sketch_basis;
  const float* sketch_scale;
  const int8_t* sketch;
  const void* vectors; /* fp16 */
  const int32_t* table;
} octexB200Arrays;

/* cuvsOctexLoad from memory instead of a directory (the reference has no such call; its loader is
 * cpp/src/neighbors/octex/load.cu:206-494). */
OCTEX_B200_EXPORT cuvsError_t octexB200Attach(cuvsResources_t res, const octexB200Arrays* arrays,
                                              cuvsOctexLoadParams_t params, int32_t rank,
                                              int32_t world, cuvsOctexIndex_t index);

/* detail::resident_search (cpp/src/neighbors/octex/search.cu:983-997): search again the queries of
 * the previous call, which are still on the GPU, and leave the results there. The timing protocol
 * of the reference's benchmark uses it (cpp/bench/octex_bench.cu:223-253). */
OCTEX_B200_EXPORT cuvsError_t octexB200SearchResident(cuvsResources_t res,
                                                      cuvsOctexSearchParams_t params,
                                                      cuvsOctexIndex_t index, int64_t n_queries,
                                                      int64_t k);

/* detail::timed_batch (search.cu:965-981) per kernel: one batch of the queries already on the GPU,
 * launched kernel by kernel with events between them. ms receives the milliseconds of centre +
 * sketch query, projection, cell codes, cell lookup, first round, (several processes, shard
 * placement: exchange of the kept lists, their merge,) each wave, best k (several processes: the
 * gathering of the results); *count their number. */
OCTEX_B200_EXPORT cuvsError_t octexB200ProfileBatch(cuvsResources_t res,
                                                    cuvsOctexSearchParams_t params,
                                                    cuvsOctexIndex_t index, int64_t n_queries,
                                                    int64_t k, float* ms, int32_t capacity,
                                                    int32_t* count);

/* Waits for the index's stream and reports, once, whether a kernel of the searches queued so far
 * gave up (the bounded waits of the tensor-core projection): CUVS_ERROR with a message, else
 * CUVS_SUCCESS. A search with host outputs checks by itself; after a search with device outputs
 * (cuvsOctexSearch on device tensors: results are only ordered on the stream of `res`,
 * c/include/cuvs/neighbors/octex.h:283-289 of the reference) this is the call that tells. */
OCTEX_B200_EXPORT cuvsError_t octexB200CheckLast(cuvsOctexIndex_t index);

/* detail::memory_report (cpp/src/neighbors/octex/search.cu:999-1016): device memory of this
 * process's GPU by index part. bytes[7] = device ordinal, copies (lists, cell tables, base), sketch,
 * table, vectors, other (projections, sketch basis, pointer tables), batch buffers of the cached
 * search configuration. Arrays kept in host memory count 0. */
OCTEX_B200_EXPORT cuvsError_t octexB200MemoryReport(cuvsOctexIndex_t index, int64_t* bytes);

/* Observation (detail::timed_batch / memory_report, search.cu:965-1016, are the reference's
 * counterparts): stats = per-query counters of what the kernels read, taps = keep the intermediate
 * arrays of the last batch. Either one changes the plan; both are off by default. */
OCTEX_B200_EXPORT cuvsError_t octexB200SetDebug(cuvsOctexIndex_t index, int32_t stats, int32_t taps);
/* The projection of the queries (the cuBLASLt call of cpp/src/neighbors/octex/search.cu:303-320)
 * runs on the tensor cores by default. ordered = 1 selects the kernel that accumulates every dot
 * product in dimension order instead, whose projected coordinates a CPU implementation can
 * reproduce bit for bit (parity tests use it); 0 goes back. Changes the plan. */
OCTEX_B200_EXPORT cuvsError_t octexB200SetProjection(cuvsOctexIndex_t index, int32_t ordered);
/* Copy a named array of the last batch to host memory: "y", "qs", "codes", "seg", "cand1",
 * "cand1_dist", "n1", "kept1_ids", "kept1_dist", "stats", "kept_ids", "kept_dist". *bytes returns
 * its size; dst may be NULL to ask for the size only. */
OCTEX_B200_EXPORT cuvsError_t octexB200Fetch(cuvsOctexIndex_t index, const char* name, void* dst,
                                             int64_t capacity, int64_t* bytes);

/* Cell codes of n rows of 8 * blocks float32 coordinates scaled by inv_f, computed on the GPU by
 * the device function every search kernel uses (e8b_hash64 of
 * cpp/src/neighbors/octex/detail/e8.cuh:66-85). Host pointers. */
OCTEX_B200_EXPORT cuvsError_t octexB200CellCodes(const float* y, int64_t n, int32_t blocks,
                                                 float inv_f, int64_t* codes);

/* Cell codes of a batch of queries, computed without allocating anything. No counterpart in the
 * reference: its search always allocates its per-batch buffers (cpp/src/neighbors/octex/search.cu
 * does so in make_plan). This call is for callers that must not allocate device memory where they
 * stand: a process whose device memory was all given to one arena at start-up (a later cudaMalloc
 * fails, or is against the rules of that process), a serving loop that cannot take the device-wide
 * synchronisation a cudaMalloc / cudaFree pair brings, and code that runs while a stream capture
 * is open elsewhere in the process, where cudaMalloc is not allowed.
 *
 * queries [n_queries, dim] float32 and codes [n_queries, copies, levels] int64 are DEVICE memory on
 * the GPU of the index, which must be the current device; the work is queued on `stream` (a
 * cudaStream_t, NULL for the default stream) and codes[q][c][j] is the code of query q's cell in
 * copy c at spacing j, every level computed. The coordinates behind these codes come from the
 * projection that sums in dimension order (octexB200SetProjection(index, 1)); they are the array
 * octexB200Fetch calls "codes" bit for bit when the search uses that projection too, which it does
 * after octexB200SetProjection(index, 1) and for every index whose copies do not have 4 blocks.
 * The default search of a 4-block index projects on the tensor cores, whose fp32 sums run in another
 * order: about 1 % of its fp16 coordinates land on the neighbouring fp16 value, so a small share of
 * its codes (a few per cent at the finest spacing) name a neighbouring cell. An index whose copies
 * are dealt over several processes (shard placement, world > 1) is refused: the call answers for
 * all copies of an index or not at all.
 *
 * The intermediates (centred fp16 queries, sketch-space queries, fp16 projected coordinates) live
 * in one fixed 32 MiB array inside the library, which every GPU that loads the library holds until
 * the process ends. A call whose n_queries * (2 * dim64 + 4 * sketch_width + 16 * blocks * copies)
 * bytes (dim64 = dim rounded up to 64) exceed 32 MiB is refused with CUVS_ERROR and a message that
 * names the largest batch that fits. All calls on a GPU share that array: it holds whatever the
 * last call left (each call overwrites every byte it later reads, nothing needs clearing), and two
 * calls that overlap on the GPU (different streams, no ordering between them) race on it. Every
 * call asks the runtime for the array's address on the current device (so the call stays valid
 * after a cudaDeviceReset); the first time that happens on a GPU the library's device code is
 * loaded there, so make the first call on each GPU outside of any stream capture. */
OCTEX_B200_EXPORT cuvsError_t octexB200QueryCodesStatic(cuvsOctexIndex_t index,
                                                        const float* queries, int64_t n_queries,
                                                        int64_t* codes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OCTEX_B200_H_ */
