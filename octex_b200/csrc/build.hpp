// The index builder's interface inside the library (the public one is octex_b200::build in
// include/octex_b200.hpp and cuvsOctexBuild in include/octex_b200.h).
#pragma once

#include "common.hpp"

#include <octex_b200.hpp>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>
#include <sys/stat.h>

namespace octex_b200 {

/// Creates the directory (and its parents) when it does not exist.
inline void make_directory(std::string const& path)
{
  std::string at;
  for (size_t i = 0; i <= path.size(); i++) {
    if (i == path.size() || path[i] == '/') {
      if (!at.empty() && at != "/") {
        if (::mkdir(at.c_str(), 0777) != 0 && errno != EEXIST) throw error("octex: cannot create " + at);
      }
    }
    if (i < path.size()) at.push_back(path[i]);
  }
  struct stat st {};
  OCTEX_EXPECTS(::stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode), "octex: " + path + " is not a directory");
}

/// The K nearest other rows of every row of x f16 [n, D] (device memory, current device) by
/// squared distance between the fp16 rows: ids i32 / dist f32 [n, K] in device memory, nearest
/// first, equal distances by ascending id, -1 / +inf where a row has fewer than K others.
/// method 0 picks the tensor-core scan when it covers the shape, 1 asks for it, 2 for the plain one.
/// Returns after the stream has finished.
void exact_neighbors(const __half* x, int64_t n, int D, int K, int method, int32_t* ids, float* dist, cudaStream_t s);

/// The neighbor table of a loaded index by the index's own search (build_table.cuh:648-841 of the
/// reference): every base row is searched for 3k/2 + 1 neighbors in passes — the first round alone,
/// then 2 and 3 waves over the table of the pass before, ranking by sketch with an exact rerank at
/// the end — the row itself is dropped and reverse edges are merged in (k/4 forward entries first,
/// up to 3k/4 reverse ones). sketch_order leaves the answers in sketch order without the exact
/// rerank (index_params::table_sketch_order). The index keeps the table of the last pass;
/// table_host (may be null) int32 [n, k] receives it. One process, fp16 rows on its GPU.
void searched_table(resources const& res, index& idx, int k, int passes, bool reverse_edges, bool sketch_order,
                    int32_t* table_host, bool verbose);

}  // namespace octex_b200
