// Launch interface of the search kernels: plain pointers and sizes, one function per kernel.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace octex_b200::kernels {

constexpr int kMinHash     = 256;    // smallest per-query hash set (slots)
constexpr int kMaxHash     = 32768;  // largest per-query hash set
constexpr int kMaxRerank   = 512;    // exact rerank depth per round
constexpr int kMaxKeepSort = 1024;   // kept + reranked keys sorted together (exact ranking)
constexpr int kMaxSketchKO = 1024;   // kept entries when ranking by sketch
constexpr int kMaxExpanded = 6144;   // start points expanded by earlier waves
constexpr int kRoundThreads = 128;  // threads of a query block unless its shared memory asks for more

/// Slots of the hash set that collects `total` entries: twelfths / 12 slots per entry (24 = half
/// full at most, 16 = three quarters), a multiple of four, between kMinHash and cap. (The reference,
/// search_kernels.cuh:33-38, takes a power of two at most two thirds full; only the memory taken and
/// the length of the probe sequences differ.)
__host__ __device__ inline int hash_slots_of(int total, int cap, int twelfths)
{
  int need = ((twelfths * total + 11) / 12 + 3) & ~3;
  if (need < kMinHash) need = kMinHash;
  return need < cap ? need : cap;
}

/// Rows [from, m) of q become copies of row 0 (padding of a partial batch).
void pad_rows(float* q, int from, int m, int D, cudaStream_t s);

/// Largest dimension center_sketch takes: its block keeps 16 centred rows in shared memory.
constexpr int kMaxDim = (227 << 10) / (16 * 4);

/// qh [m, ldq] = half(q - mean) zero-padded to ldq columns; qs [m, S] = (q - mean) @ basis in fp32
/// (one fused multiply-add per dimension, in dimension order).
void center_sketch(const float* q, const float* mean, const float* basis, int m, int D, int S,
                   __half* qh, int ldq, float* qs, cudaStream_t s);

/// Y [m, N] = half(fp32(qh . ut^T) + shift) with the dot product accumulated by one fused
/// multiply-add per dimension in dimension order (the order of the CPU checker). ut is [N, ldu].
void project_ordered(const __half* qh, int ldq, const __half* ut, int ldu, const __half* shift,
                     int m, int N, int D, __half* Y, cudaStream_t s);

/// codes [pairs, L] = cell code at every level of the 8*blocks coordinates of each (query, copy)
/// pair of Y [pairs, 8*blocks]. level_on [C, L] (may be null) marks the levels that hold cells;
/// the others get code 0 and are never looked at.
void decode_codes(const __half* Y, int64_t pairs, int C, int blocks, int L, const float* inv_f,
                  const unsigned char* level_on, long long* codes, cudaStream_t s);

/// Tensor-core projection with the decode in its epilogue (project_tc.cu): TMA tensor maps of the
/// two operands, made once per plan.
struct project_tc_plan {
  alignas(64) unsigned char map_a[128];  // fp16 queries [m, ldu]
  alignas(64) unsigned char map_b[128];  // fp16 projections [copies * 32, ldu]
  int m = 0, copies = 0, ldu = 0;
};
/// The cell lookup done inside the projection's epilogue (table == nullptr: not done there; the
/// codes are written out for the separate kernel instead). Needs level_on.
struct cell_slot;
struct tc_lookup {
  const cell_slot* table = nullptr;
  const long long* toff  = nullptr;
  const int* tmask       = nullptr;
  const int* base        = nullptr;
  int list_len = 0, lr = 0;
  int2* seg        = nullptr;  // [m, copies]
  long long* stats = nullptr;  // [m, 8] += (levels tried, slots examined), may be null
};
/// True when the tensor-core kernel covers this index shape (4 blocks per copy).
bool project_tc_supported(int blocks, int ldu);
void project_tc_setup(project_tc_plan& p, const __half* qh, int m, const __half* ut, int copies, int ldu);
/// codes [m, copies, L] (and Yout [m, copies * 32] fp16 when not null) from the operands of the
/// plan. *error (device-visible int) becomes non-zero when a wait inside the kernel ran out.
/// finest = the smallest spacing (host copy): coordinates small against it take the short decode.
/// With look.table set, the lookup of the cells happens in the same kernel: seg is written, codes
/// is not.
void project_decode_tc(const project_tc_plan& p, int L, const __half* shift, const float* inv_f,
                       float finest, const unsigned char* level_on, long long* codes, __half* Yout,
                       const tc_lookup& look, int* error, cudaStream_t s);

/// codes [n] = cell code of each row of y [n, 8*blocks] float32 scaled by inv_f.
void cell_codes_f32(const float* y, int64_t n, int blocks, float inv_f, long long* codes,
                    cudaStream_t s);

/// One slot of the cell table of a (copy, level): the 64-bit code of a cell and the row of its list
/// among the level's cells (-1: empty slot). 16 bytes: a lookup reads one 32-byte sector, where the
/// reference's bucket array plus key array (detail/search_kernels.cuh:100-126) costs two dependent
/// ones.
struct cell_slot {
  long long key;
  int row;
  int pad;
};

/// Fill the open-addressing tables of CL (copy, level) pairs from their key arrays: pair cl holds
/// ncells[cl] codes keys[cl * mmax + p], p = row of the cell; its table is table + toff[cl],
/// tmask[cl] + 1 slots (a power of two, at least twice the cells), home slot = low bits of the code.
/// The table must be filled with 0xff bytes before (row -1 everywhere).
void build_cell_tables(const long long* keys, int64_t mmax, const int* ncells, const long long* toff,
                       const int* tmask, int CL, cell_slot* table, cudaStream_t s);

/// seg [m, C] = (first list entry, entries read) of the finest level whose cell holds a list,
/// (0, 0) when none does. stats (may be null) [m, 2] += (levels tried, table slots examined).
void probe(const long long* codes, int m, int C, int L, const cell_slot* table, const long long* toff,
           const int* tmask, const int* base, const unsigned char* level_on, int list_len, int lr,
           int2* seg, long long* stats, cudaStream_t s);

/// norm [rows] = sum_k (code_k * scale_k)^2 of each row of codes [rows, S] as fp32 (one fused
/// multiply-add per code, in code order): the part of the sketch distance that depends on the row
/// alone. All device memory.
void sketch_row_norms(const signed char* codes, const float* scale, int64_t rows, int S, float* norm,
                      cudaStream_t s);

/// Where the rows of an array live when they are dealt over the GPUs in ranges of `rows`
/// (ptrs[g] = start of rows [g * rows, (g + 1) * rows) in that GPU's memory, mapped into this
/// process); ptrs == nullptr: the whole array is behind the plain pointer. The reference's
/// xptr / cptr / tptr tables with xrows / crows (detail/search_kernels.cuh:40-55).
struct row_map {
  const long long* ptrs = nullptr;
  int rows              = 0;
  int local             = 0;  // a row this GPU holds itself (stand-in where a lane has no row to read)
};

/// One round of a query block: distinct ids of its segments, sketch distances, the R nearest by
/// sketch reranked exactly (or the KO nearest kept by sketch distance), merged into the kept list.
struct round_args {
  int m = 0;     // queries = thread blocks
  int nseg = 0;  // segments per query: copies (lists) or starts (table rows)
  // lists mode: segment (start, len) into the lists of copy c
  const int2* seg = nullptr;
  const int* lists = nullptr;
  int64_t stride = 0;
  int lr = 0;  // entries read per non-empty segment (every segment is 0 or lr long)
  // rows mode: the first `starts` kept entries no earlier wave expanded; their table rows
  const int* table = nullptr;
  int table_len = 0;
  int* done = nullptr;  // [m, done_stride] start points of all waves
  int done_stride = 0;
  int done_off = 0;  // entries of earlier waves
  int pick_slots = 0;  // hash slots for the earlier start points (power of two)
  // sketch: rows of sw codes; sketch_norm [n]: the constant of every row (sketch_row_norms),
  // whole on every GPU even when the rows are dealt
  const signed char* sketch = nullptr;
  const float* sketch_norm = nullptr;
  const float* scale = nullptr;
  const float* qs = nullptr;  // [m, sw]
  int sw = 0;
  // exact rerank
  const __half* vectors = nullptr;
  int D = 0;
  const float* Q = nullptr;  // [m, D] uncentred queries
  int R = 0;                 // rerank depth (exact) — ignored when sketch_rank
  int KO = 0;
  int sketch_rank = 0;
  int fresh = 0;  // the kept list starts empty
  long long* si = nullptr;  // kept ids [m, KO]
  float* sd = nullptr;      // kept distances [m, KO]
  // sizes of the shared-memory carve-up (host decides)
  int ht_slots = 0;   // ints of the hash set region (>= largest set used, >= pick_slots)
  int cap_slots = 0;  // largest gather hash set (slots)
  int hash_twelfths = 16;  // slots per 12 gathered entries (host: as sparse as shared memory allows)
  int keep_sketch = 0;  // the sketch and its row constants fit the L2 cache with room to spare: load them
                        // with an evict-last policy, the large arrays with evict-first (host decides)
  int threads = kRoundThreads;  // threads per query block: 128, 256 or 512 (host: the smallest
                                // that still fills a multiprocessor with the blocks that fit it)
  int nmax = 0;       // capacity of the candidate / distance arrays
  int P = 0;          // keys sorted by the merge (power of two >= KO)
  int* cand_global = nullptr;    // [m, nmax] when the candidates do not fit shared memory
  float* dist_global = nullptr;  // [m, nmax] when the region of the hash set (ht_slots) cannot hold them
  // rows dealt over GPUs (all empty: every array is whole behind its pointer)
  row_map table_map, sketch_map, vector_map;
  // observation (all may be null)
  int* tap_cand = nullptr;    // [m, tap_cap]
  float* tap_dist = nullptr;  // [m, tap_cap]
  int* tap_n = nullptr;       // [m]
  int tap_cap = 0;
  long long* phase = nullptr;  // [m, 8] cycles per phase of the block (observation)
  long long* stats = nullptr;  // [m, 8]: [2] entries read, [3] distinct ids first round,
                               // [4] table rows expanded, [5] distinct ids of waves,
                               // [6] rows selected for the exact rerank, [7] of them read
                               // (a selected id already in the kept list is not read again)
};
size_t round_smem_bytes(const round_args& a);
void round_lists(const round_args& a, cudaStream_t s);
void round_rows(const round_args& a, cudaStream_t s);
/// Opt every round kernel in to `bytes` of dynamic shared memory on the current device.
void round_allow_smem(size_t bytes);

/// bi, bd [m, k] = the first k columns of si, sd [m, KO].
void take_k(const long long* si, const float* sd, int KO, int k, int m, long long* bi, float* bd,
            cudaStream_t s);

/// Exact rerank of the first R kept entries (sketch ranking) into the best k.
void final_rerank(const long long* si, int KO, int R, const __half* vectors, row_map vector_map, int D,
                  const float* Q, int k, int m, long long* bi, float* bd, long long* stats,
                  cudaStream_t s);

/// Merge of nsrc kept lists [*, KO] (already in this GPU's memory, back to back: source h at
/// src + h * src_stride): nearest copy of every id, best KO.
void merge_kept(const long long* src_i, const float* src_d, int nsrc, int64_t src_stride, int KO,
                int P, int m, long long* si, float* sd, cudaStream_t s);

/// Exact K nearest rows (self excluded) of the rows [q_first, q_first + q_count) of x f16 [n, D]
/// among all n rows, by |a|^2 + |b|^2 - 2 a.b with the dot products on the tensor cores
/// (knn_tc.cu); norm f32 [n] = |x_r|^2. best_id i32 / best_d f32 [q_count, K], nearest first,
/// equal distances by ascending id, -1 / +inf padded. *error (device word, zero on entry) is set
/// when a wait inside the kernel ran out; the lists are then incomplete.
bool knn_tc_supported(int64_t n, int D, int K);
void knn_tc(const __half* x, const float* norm, int64_t n, int D, int K, int64_t q_first, int64_t q_count,
            int32_t* best_id, float* best_d, int* error, cudaStream_t s);

}  // namespace octex_b200::kernels
