/* TEST INFRASTRUCTURE ONLY: C interface of the CPU restatement of the octex batched search.
 * Only tests/, the smoke check and the CPU-baseline leg of the benchmark may load it. */
#ifndef OCTEX_ORACLE_H_
#define OCTEX_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The arrays of an index directory (format 1), all in host memory, as the files hold them. */
typedef struct {
  int64_t n, dim;
  int32_t copies, blocks, levels, list_len, log_buckets, sketch_width, table_len, pad_;
  int64_t stride;          /* entries per copy in lists */
  int64_t mmax;            /* keys per (copy, level) */
  const float* spacings;   /* [levels] */
  const float* mean;       /* [dim] */
  const float* proj;       /* [copies, dim, 8*blocks] */
  const float* shift;      /* [copies, 8*blocks] */
  const int32_t* lists;    /* [copies, stride] */
  const int64_t* keys;     /* [copies, levels, mmax] */
  const int32_t* offsets;  /* [copies, levels, 2^log_buckets + 1] */
  const int32_t* base;     /* [copies, levels] */
  const float* basis;      /* [dim, sketch_width] */
  const float* scale;      /* [sketch_width] */
  const int8_t* sketch;    /* [n, sketch_width] */
  const uint16_t* vectors; /* [n, dim] fp16 bit patterns */
  const int32_t* table;    /* [n, table_len], -1 padded; NULL when table_len == 0 */
} oracle_index;

typedef struct {
  int32_t read, starts, waves, rerank, wave_rerank, batch;
  int32_t sketch_rank, final_rerank;
  int32_t parts;   /* GPUs of a sharded placement emulated (1: no cross-part merge) */
  int32_t threads; /* host threads (0: all) */
  int32_t sketch_form; /* 0: the sketch distance as the CUDA path computes it: the integer form
                          (sketch_distance_int in octex_oracle.cpp) in the first round of a search
                          that reranks exactly, the fp32 sum (code * scale - q)^2 otherwise;
                          1: the fp32 sum in every round, the reference's own terms */
} oracle_params;

/* Optional observation points; any pointer may be NULL. */
typedef struct {
  const uint16_t* y_in; /* [nq, copies*8*blocks] fp16: use these projected coordinates */
  uint16_t* y;          /* [nq, copies*8*blocks] fp16 projected coordinates used */
  float* qs;            /* [nq, sketch_width] sketch-space queries */
  int64_t* codes;       /* [nq, copies, levels] cell codes (all levels) */
  int32_t* seg;         /* [nq, copies, 2] (first list entry, entries read) */
  int32_t* cand1;       /* [nq, cand_cap] distinct first-round ids, ascending, part 0.. concatenated */
  float* cand1_dist;    /* [nq, cand_cap] their sketch distances */
  int32_t* n1;          /* [nq] count of cand1 */
  int32_t cand_cap, pad_;
  int64_t* kept1_ids;   /* [nq, KO] kept list after the first round (merged over parts) */
  float* kept1_dist;    /* [nq, KO] */
  int64_t* stats;       /* [nq, 8]: levels tried, keys scanned, list entries read, n1,
                           table rows expanded, sum of n2, rows reranked exactly, unused */
} oracle_taps;

/* Error text of the last failing call of this thread ("" when none). */
const char* oracle_last_error(void);

/* nearest E8 point of each of n_blocks groups of 8 floats */
int oracle_e8_point(const float* x, int64_t n_blocks, float* p);
/* cell code of each of n rows of 8*b floats scaled by inv_f */
int oracle_cell_code(const float* y, int64_t n, int32_t b, float inv_f, int64_t* h);
/* float -> fp16 bit patterns (round to nearest even) and back */
int oracle_to_half(const float* x, int64_t n, uint16_t* h);
int oracle_from_half(const uint16_t* h, int64_t n, float* x);

/* Whole search of nq queries [nq, dim]; neighbors int64 [nq, k], distances float [nq, k]. */
int oracle_search(const oracle_index* ix,
                  const oracle_params* sp,
                  const float* queries,
                  int64_t nq,
                  int32_t k,
                  int64_t* neighbors,
                  float* distances,
                  const oracle_taps* taps);

/* Exact brute-force k nearest by squared L2 in float64 over fp32 rows (ground truth). */
int oracle_brute_force(const float* base, int64_t n, int64_t dim, const float* queries, int64_t nq,
                       int32_t k, int32_t threads, int64_t* ids, float* dist);

#ifdef __cplusplus
}
#endif
#endif
