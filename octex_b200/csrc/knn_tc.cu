// Exact K nearest rows of every row of an fp16 matrix, on the tensor cores (sm_100a only): what the
// neighbor table of an index is made from (the reference calls cuVS brute force for it: hpdic/octex,
// cpp/src/neighbors/octex/detail/build_table.cuh:60-142).
//
//   t[q, r] = |x_r|^2 - 2 x_q . x_r          squared distance up to the row's own constant |x_q|^2
//
// A block owns 128 query rows and walks over all rows in tiles of 128. Per tile the 128 x 128 dot
// products are one tcgen05.mma chain (fp16 operands by TMA, 128-byte swizzle, fp32 accumulators in
// TMEM); the accumulators are double buffered, so the tensor cores work on tile i + 1 while the
// epilogue warps read tile i out of TMEM (tcgen05.ld, one query row per thread), add the row norms
// and compare against the worst entry the row keeps. A row meets about K (1 + ln(n / K))
// improvements in all, so after the first few tiles the epilogue is one fused multiply-add and a
// fraction of a comparison per element. A thread only notes an improvement (value, row) in a
// small buffer; after every 32 columns the warp empties the buffers of its 32 rows together: the
// new entry replaces the worst of the row's list in shared memory and the lanes look for the new
// worst with warp-wide maximum instructions. The lists are put in order once, at the end.
// Nothing in the loop calls a function or touches the stack: with nearly all of the L1 given to
// shared memory, a call's spills would go to the L2 cache and cost more than the tile.
//
// Roles: warp 0 issues the TMA copies, warp 1 the MMAs (one lane each); the other warps are the
// epilogue, in sets of four (one per quarter of the TMEM lanes). With two sets (short lists only:
// each set keeps its own list per row, merged at the end) the tiles alternate between them.
// Every wait on an mbarrier is bounded; a wait that runs out raises a flag the other roles see, the
// block waits for its copies in flight, frees its TMEM and returns with the error word set.

#include "kernels.hpp"

#include "tc_common.cuh"

#include <algorithm>

namespace octex_b200::kernels {

namespace {

constexpr int kTile       = 128;  // query rows per block = rows per tile = TMEM lanes
constexpr int kKnnThreads = 320;  // at most: copy warp, MMA warp, two sets of four epilogue warps
constexpr int kTmemCols   = 256;  // two accumulators of 128 fp32 columns
constexpr uint32_t kStageBytes = 2 * kTile * kTileK * 2;  // A and B tile of a stage

struct knn_ctl {
  uint64_t full[4], empty[4];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int failed;
  alignas(16) float nb[8][kTile];  // norms of the rows of the tile an epilogue warp works on
  int state[2][kTile][2];          // per set and query row: entries kept at the end of the scan
};
constexpr int kCtlBytes = 8192;
constexpr int kNoted    = 32;  // improvements a row can note between two visits of its warp (32 columns)

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Both TMEM instructions are warp-wide: the lanes meet first (a scan before them may have diverged).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
  __syncwarp();
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
      "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
      "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
      "=r"(r[30]), "=r"(r[31])
    : "r"(taddr)
    : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
  __syncwarp();
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


__global__ void __launch_bounds__(kKnnThreads, 1)
  knn_tc_kernel(const __grid_constant__ CUtensorMap map, const float* __restrict__ norm, int64_t n, int nkb,
                int K, int stages, int64_t q_first, int64_t q_count, int32_t* __restrict__ best_id,
                float* __restrict__ best_d, int* __restrict__ error)
{
  extern __shared__ unsigned char raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t{1023});
  __half* tiles       = reinterpret_cast<__half*>(base);  // [stages][A 128 x 64 | B 128 x 64]
  knn_ctl& ctl        = *reinterpret_cast<knn_ctl*>(base + static_cast<size_t>(stages) * kStageBytes);
  float* lists        = reinterpret_cast<float*>(base + static_cast<size_t>(stages) * kStageBytes + kCtlBytes);
  static_assert(sizeof(knn_ctl) <= kCtlBytes, "control block");
  const int sets = (static_cast<int>(blockDim.x) - 64) / 128;  // sets of four epilogue warps: 1 or 2

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t q0     = q_first + static_cast<int64_t>(blockIdx.x) * kTile;
  const int64_t ntiles = (n + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 4; s++) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&ctl.acc_full[b], 1);
      mbar_init(&ctl.acc_empty[b], 4);  // one arrival per epilogue warp
    }
    ctl.failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem      = ctl.tmem_base;
  const volatile int* stop = &ctl.failed;

  if (warp == 0) {
    // ---- copies ------------------------------------------------------------------------------
    if (lane == 0) {
      bool ok    = true;
      int64_t it = 0;
      for (int64_t t = 0; t < ntiles && ok; t++) {
        for (int kb = 0; kb < nkb; kb++, it++) {
          const int s       = static_cast<int>(it % stages);
          const uint32_t ph = static_cast<uint32_t>(it / stages) & 1u;
          if (it >= stages) ok = mbar_wait(&ctl.empty[s], ph ^ 1u, stop);
          if (!ok) break;
          __half* a = tiles + static_cast<size_t>(s) * (kStageBytes / 2);
          mbar_expect_tx(&ctl.full[s], kStageBytes);
          tma_load_2d(a, &map, kb * kTileK, static_cast<int>(q0), &ctl.full[s]);
          tma_load_2d(a + kTile * kTileK, &map, kb * kTileK, static_cast<int>(t * kTile), &ctl.full[s]);
        }
      }
      if (!ok && atomicExch(&ctl.failed, 1) == 0) atomicExch(error, 1);
    }
  } else if (warp == 1) {
    // ---- MMAs --------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(kTile >> 3) << 17) |
                                 (static_cast<uint32_t>(kTile >> 4) << 24);
      bool ok    = true;
      int64_t it = 0;
      for (int64_t t = 0; t < ntiles && ok; t++) {
        const int b      = static_cast<int>(t & 1);
        const uint32_t u = static_cast<uint32_t>(t >> 1);
        if (t >= 2) ok = mbar_wait(&ctl.acc_empty[b], (u & 1u) ^ 1u, stop);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < nkb; kb++, it++) {
          const int s       = static_cast<int>(it % stages);
          const uint32_t ph = static_cast<uint32_t>(it / stages) & 1u;
          ok = mbar_wait(&ctl.full[s], ph, stop);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const __half* a   = tiles + static_cast<size_t>(s) * (kStageBytes / 2);
          const uint64_t da = umma_desc(a), db = umma_desc(a + kTile * kTileK);
#pragma unroll
          for (int k = 0; k < kTileK / 16; k++)
            umma_f16(tmem + static_cast<uint32_t>(b * kTile), da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&ctl.empty[s]);  // arrives when the MMAs reading this stage are done
        }
        if (ok) umma_commit(&ctl.acc_full[b]);
      }
      if (!ok && atomicExch(&ctl.failed, 1) == 0) atomicExch(error, 2);
    }
  } else {
    // ---- epilogue: one query row per thread, the tiles dealt over the sets of four warps --------
    const int quarter = warp & 3;  // the TMEM lanes this warp may read
    const int e       = quarter * 32 + lane;
    const int ew      = warp - 2;
    const int set     = ew >> 2;
    const int64_t row = q0 + e;
    const bool live   = row < q_first + q_count && row < n;
    // lists: values [set][row][K], then ids alike; noted improvements: values [set][slot][row], ids alike
    float* values = lists;
    int32_t* ids  = reinterpret_cast<int32_t*>(lists + static_cast<size_t>(sets) * kTile * K);
    auto list_of  = [&](int of_set, int of_row) { return (static_cast<size_t>(of_set) * kTile + of_row) * K; };
    float* noted_d   = reinterpret_cast<float*>(ids + static_cast<size_t>(sets) * kTile * K) + static_cast<size_t>(set) * kNoted * kTile + e;
    int32_t* noted_i = reinterpret_cast<int32_t*>(lists + static_cast<size_t>(sets) * kTile * (2 * K + kNoted)) +
                       static_cast<size_t>(set) * kNoted * kTile + e;
    float* ld    = values + list_of(set, quarter * 32);  // the lists of the warp's 32 rows
    int32_t* li  = ids + list_of(set, quarter * 32);
    float kth    = live ? INFINITY : -INFINITY;  // what a row has to beat: the worst kept, once the list is full
    int have     = live ? 0 : K;                  // entries the row's list holds
    int worst    = 0;                             // slot of the worst one
    int noted    = 0;                             // improvements noted since the warp last took them in
    float* nb    = ctl.nb[ew];
    // 32 columns of the tile: note what beats the row's bar, then the warp takes in what its lanes
    // noted, a row at a time. The tile loop calls this from one place (a rolled loop over the four
    // quarters of the columns): the loop has to stay small, its warp is alone on its scheduler and
    // nothing hides an instruction fetch.
    auto scan = [&](const uint32_t (&r)[32], int col, int64_t first) {
      float d[32];
#pragma unroll
      for (int g = 0; g < 8; g++) {
        const float4 nn = *reinterpret_cast<const float4*>(nb + col + g * 4);
        d[g * 4 + 0]    = fmaf(-2.f, __uint_as_float(r[g * 4 + 0]), nn.x);
        d[g * 4 + 1]    = fmaf(-2.f, __uint_as_float(r[g * 4 + 1]), nn.y);
        d[g * 4 + 2]    = fmaf(-2.f, __uint_as_float(r[g * 4 + 2]), nn.z);
        d[g * 4 + 3]    = fmaf(-2.f, __uint_as_float(r[g * 4 + 3]), nn.w);
      }
      float m[16];
#pragma unroll
      for (int i = 0; i < 16; i++)
        m[i] = fminf(d[i], d[i + 16]);
#pragma unroll
      for (int w = 8; w > 0; w >>= 1)
#pragma unroll
        for (int i = 0; i < w; i++)
          m[i] = fminf(m[i], m[i + w]);
      const float least = m[0];
      if (least < kth) {  // rare
#pragma unroll
        for (int i = 0; i < 32; i++)
          if (d[i] < kth) {
            noted_d[noted * kTile] = d[i];
            noted_i[noted * kTile] = static_cast<int32_t>(first + i);
            noted++;  // at most 32 between two visits of the warp: kNoted slots
          }
      }
      unsigned has = __ballot_sync(0xffffffffu, noted > 0);
      while (has != 0) {
        const int L = __ffs(has) - 1;
        has &= has - 1;
        const int count = __shfl_sync(0xffffffffu, noted, L);
        float beat      = __shfl_sync(0xffffffffu, kth, L);
        int kept        = __shfl_sync(0xffffffffu, have, L);
        int slot        = __shfl_sync(0xffffffffu, worst, L);
        float* vd       = ld + static_cast<size_t>(L) * K;
        int32_t* vi     = li + static_cast<size_t>(L) * K;
        for (int j = 0; j < count; j++) {
          const float dj   = noted_d[j * kTile + (L - lane)];  // row L's slot j: the same word for every lane
          const int32_t id = noted_i[j * kTile + (L - lane)];
          if (!(dj < beat) || id == q0 + quarter * 32 + L) continue;
          // the new entry takes a free slot or the worst one's
          const int at = kept < K ? kept : slot;
          if (lane == 0) {
            vd[at] = dj;
            vi[at] = id;
          }
          if (kept < K) kept++;
          __syncwarp();
          if (kept < K) continue;  // still filling: everything gets in
          // the worst kept, the largest (value, id): rows arrive by ascending id, so of equal values
          // the later row is the worse one and a row equal to the worst never gets in
          unsigned bk = 0;
          int32_t bi  = -1;
          int bs      = 0;
          for (int t = lane; t < K; t += 32) {
            const unsigned u = __float_as_uint(vd[t]);
            const unsigned k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // same order as the floats
            const int32_t i  = vi[t];
            if (k > bk || (k == bk && i > bi)) {
              bk = k;
              bi = i;
              bs = t;
            }
          }
          const unsigned top  = __reduce_max_sync(0xffffffffu, bk);
          const int32_t last  = __reduce_max_sync(0xffffffffu, bk == top ? bi : -1);
          const unsigned owns = __ballot_sync(0xffffffffu, bk == top && bi == last);
          slot                = __shfl_sync(0xffffffffu, bs, __ffs(owns) - 1);
          beat                = __uint_as_float((top & 0x80000000u) ? (top & 0x7fffffffu) : ~top);
          __syncwarp();
        }
        if (lane == L) {
          kth   = beat;
          have  = kept;
          worst = slot;
          noted = 0;
        }
      }
    };
    // norms of the rows of a tile, four per lane; rows beyond the matrix never win
    auto fetch_norms = [&](int64_t t, float (&v)[4]) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int64_t r = t * kTile + i * 32 + lane;
        v[i]            = (t < ntiles && r < n) ? __ldg(norm + r) : INFINITY;
      }
    };
    float ahead[4];
    fetch_norms(set, ahead);
    bool ok = true;
    for (int64_t t = set; t < ntiles; t += sets) {
      const int b      = static_cast<int>(t & 1);
      const uint32_t u = static_cast<uint32_t>(t >> 1);
      const int64_t r0 = t * kTile;
      __syncwarp();  // every lane is done with the norms of the warp's previous tile
#pragma unroll
      for (int i = 0; i < 4; i++)
        nb[i * 32 + lane] = ahead[i];
      fetch_norms(t + sets, ahead);  // for the warp's next tile: in flight behind this one
      __syncwarp();
      ok = mbar_wait(&ctl.acc_full[b], u & 1u, stop);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(b * kTile);
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t r[32];
        tmem_ld32(taddr + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
        if (c == 3) {
          // the accumulator is in registers: the tensor cores may overwrite it
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.acc_empty[b]);
        }
        scan(r, c * 32, r0 + c * 32);
      }
    }
    ctl.state[set][e][0] = live ? have : 0;
    if (!ok && lane == 0 && atomicExch(&ctl.failed, 1) == 0) atomicExch(error, 3);
    // the sets meet; the warps of the first one put the lists of their rows in order, a row at a
    // time: an entry's place is the number of entries before it by (value, id)
    asm volatile("bar.sync 1, %0;" ::"r"(sets * 128) : "memory");
    if (set == 0 && *stop == 0) {
      for (int L = 0; L < 32; L++) {
        const int of_row  = quarter * 32 + L;
        const int64_t qr  = q0 + of_row;
        if (!(qr < q_first + q_count && qr < n)) continue;
        const int have0   = ctl.state[0][of_row][0];
        const int total   = have0 + (sets == 2 ? ctl.state[1][of_row][0] : 0);
        const size_t at0  = list_of(0, of_row), at1 = list_of(sets - 1, of_row);
        auto entry = [&](int j, float& v, int32_t& id) {
          const size_t w = j < have0 ? at0 + j : at1 + (j - have0);
          v  = values[w];
          id = ids[w];
        };
        const float qn = __ldg(norm + qr);
        int32_t* oi    = best_id + (qr - q_first) * K;
        float* od      = best_d + (qr - q_first) * K;
        for (int j = lane; j < total; j += 32) {
          float v, w;
          int32_t id, other;
          entry(j, v, id);
          int place = 0;
          for (int t = 0; t < total; t++) {
            entry(t, w, other);
            place += (w < v || (w == v && other < id)) ? 1 : 0;
          }
          if (place < K) {
            oi[place] = id;
            od[place] = fmaxf(__fadd_rn(qn, v), 0.f);
          }
        }
        for (int t = total + lane; t < K; t += 32) {
          oi[t] = -1;
          od[t] = INFINITY;
        }
      }
    }
  }
  __syncwarp();
  if (*stop != 0) {
    // let the copies this block still has in flight land before its shared memory goes away
    for (int i = 0; i < 2048; i++)
      __nanosleep(512);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

size_t knn_smem_bytes(int K, int stages, int sets)
{
  return 1024 + static_cast<size_t>(stages) * kStageBytes + kCtlBytes + static_cast<size_t>(sets) * (K + kNoted) * kTile * 8;
}

/// Two sets of epilogue warps (each keeps a list per row, merged at the end) when their lists
/// leave room for two stages of operands; else one set with as many stages as fit.
void knn_shape(int K, int& stages, int& sets)
{
  for (sets = 2; sets >= 1; sets--)
    for (stages = sets == 2 ? 3 : 4; stages >= 2; stages--)
      if (knn_smem_bytes(K, stages, sets) <= 227 * 1024) return;
  stages = 0;
  sets   = 0;
}

}  // namespace

bool knn_tc_supported(int64_t n, int D, int K)
{
  // rows must start on 16-byte boundaries for the tensor map; ids are 32-bit
  int stages = 0, sets = 0;
  knn_shape(K, stages, sets);
  return D % 8 == 0 && K >= 1 && stages >= 2 && n < (int64_t{1} << 31) - kTile;
}

void knn_tc(const __half* x, const float* norm, int64_t n, int D, int K, int64_t q_first, int64_t q_count,
            int32_t* best_id, float* best_d, int* error, cudaStream_t s)
{
  if (q_count <= 0 || n <= 0) return;
  if (!knn_tc_supported(n, D, K)) throw std::runtime_error("octex: shape not covered by the tensor-core neighbor scan");
  CUtensorMap map;
  make_map(&map, x, n, D, kTile);
  int stages = 0, sets = 0;
  knn_shape(K, stages, sets);
  const size_t smem  = knn_smem_bytes(K, stages, sets);
  cudaError_t status = cudaFuncSetAttribute(knn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (status != cudaSuccess) throw std::runtime_error(std::string("octex: ") + cudaGetErrorString(status));
  const int64_t blocks = (q_count + kTile - 1) / kTile;
  knn_tc_kernel<<<static_cast<unsigned>(blocks), 64 + 128 * sets, smem, s>>>(map, norm, n, (D + kTileK - 1) / kTileK, K, stages,
                                                                         q_first, q_count, best_id, best_d, error);
}

}  // namespace octex_b200::kernels
