// Projection of a query batch on all copies with the E8 decode in the epilogue (sm_100a only):
//   acc[m, Cg*32] = qh[m, K] . ut[Cg*32, K]^T        tcgen05.mma, fp16 in, fp32 accumulators in TMEM
//   y = half(acc + shift)                             what the reference's GEMM writes out
//   codes[q, c, j] = cell code of y[q, c*32 .. c*32+32) at spacing j
//
// Answers the cuBLASLt call of the reference (hpdic/octex, cpp/src/neighbors/octex/search.cu:139-168,
// 303-320: fp16 operands, fp32 accumulate, fp16 bias epilogue, fp16 output) and the decode half of
// its probe_kernel (detail/search_kernels.cuh:100-114). The projected coordinates never go to
// memory: a thread of the epilogue owns one query row, reads the 32 accumulator columns of one
// copy from TMEM (tcgen05.ld 32x32b.x32 hands a lane exactly one copy), rounds them to fp16 and
// decodes every populated spacing.
//
// One 128 x 128 output tile per block of 256 threads. Operand tiles of 128 rows x 64 halves
// (128 bytes, the swizzle span) come in by TMA (cp.async.bulk.tensor, no cluster forms) into a
// two-stage ring; one thread issues the copies and the MMAs; every wait on an mbarrier is bounded
// and a wait that runs out sets an error word, lets the block free its TMEM and return.

#include "kernels.hpp"

#include "e8.cuh"
#include "tc_common.cuh"

#include <cstring>

namespace octex_b200::kernels {

namespace {

constexpr int kTileM    = 128;  // queries per tile = TMEM lanes
constexpr int kTileN    = 128;  // projected coordinates per tile = 4 copies of 32
constexpr int kStages   = 2;
constexpr int kThreads  = 256;  // two warps per TMEM lane quarter, each decoding half of the copies
constexpr int kTmemCols = 128;  // fp32 accumulator columns
constexpr uint32_t kStageBytes = (kTileM + kTileN) * kTileK * 2;

struct __align__(1024) tc_smem {
  __half a[kStages][kTileM * kTileK];
  __half b[kStages][kTileN * kTileK];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t done;
  uint32_t tmem_base;
  int failed;
  float shift[kTileN];
  float inv_f[16];
};

// Two blocks per SM: the decode keeps 32 coordinates and its intermediates in registers without
// spilling at 128 registers per thread, which beats three blocks at 80 with spills.
__global__ void __launch_bounds__(kThreads, 2) project_decode_tc_kernel(
  const __grid_constant__ CUtensorMap map_a,
  const __grid_constant__ CUtensorMap map_b,
  int m,
  int Cg,
  int L,
  int nkb,
  const __half* __restrict__ shift,
  const float* __restrict__ inv_f,
  float tame_y,
  const unsigned char* __restrict__ level_on,
  long long* __restrict__ codes,
  __half* __restrict__ Yout,
  const tc_lookup look,
  int* __restrict__ error)
{
  extern __shared__ unsigned char raw[];
  tc_smem& sm = *reinterpret_cast<tc_smem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t{1023});
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.y;
  const int N      = Cg * 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.done, 1);
    sm.failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < kTileN; i += kThreads) {
    const int col = tile_n * kTileN + i;
    sm.shift[i]   = col < N ? __half2float(shift[col]) : 0.f;
  }
  if (threadIdx.x < L) sm.inv_f[threadIdx.x] = inv_f[threadIdx.x];
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;

  if (threadIdx.x == 0) {
    // instruction descriptor: D fp32, A and B fp16, both K-major, N = 128, M = 128
    constexpr uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
                               (static_cast<uint32_t>(kTileM >> 4) << 24);
    auto load_stage = [&](int kb) {
      const int s = kb % kStages;
      mbar_expect_tx(&sm.full[s], kStageBytes);
      tma_load_2d(sm.a[s], &map_a, kb * kTileK, tile_m * kTileM, &sm.full[s]);
      tma_load_2d(sm.b[s], &map_b, kb * kTileK, tile_n * kTileN, &sm.full[s]);
    };
    for (int kb = 0; kb < min(nkb, kStages); kb++)
      load_stage(kb);
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; kb++) {
      const int s          = kb % kStages;
      const uint32_t phase = (kb / kStages) & 1;
      ok                   = mbar_wait(&sm.full[s], phase);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t da = umma_desc(sm.a[s]), db = umma_desc(sm.b[s]);
#pragma unroll
      for (int k = 0; k < kTileK / 16; k++)  // 16 halves = 32 bytes = 2 descriptor units per step
        umma_f16(tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
      if (kb + kStages < nkb) {
        umma_commit(&sm.empty[s]);  // arrives when the MMAs reading this stage are done
        ok = mbar_wait(&sm.empty[s], phase);
        if (ok) load_stage(kb + kStages);
      }
    }
    if (ok) {
      umma_commit(&sm.done);
    } else {
      sm.failed = 1;
      atomicExch(error, 1);
    }
  }
  __syncwarp();
  // everybody waits for the accumulators (or for the failure mark the issuing thread leaves)
  const bool ready = mbar_wait(&sm.done, 0, &sm.failed);
  if (!ready && threadIdx.x == 0) atomicExch(error, 2);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncwarp();

  // warp w reads TMEM lanes 32 (w % 4) .. + 31; warps 0-3 take the first half of the tile's copies,
  // warps 4-7 the second
  const int quarter = warp & 3;
  const int row     = tile_m * kTileM + quarter * 32 + lane;
  constexpr int kHalf = kTileN / 32 / 2;
  for (int cc = (warp >> 2) * kHalf; cc < (warp >> 2) * kHalf + kHalf; cc++) {
    __syncwarp();  // the TMEM load below is a warp-wide instruction
    uint32_t r[32];
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(cc * 32);
    asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    const int c = tile_n * (kTileN / 32) + cc;
    if (!ready || row >= m || c >= Cg) continue;
    float y[32];
    __align__(16) __half yh[32];
    bool wild = false;  // a coordinate too large for the short decode (or not a number)
#pragma unroll
    for (int i = 0; i < 32; i++) {
      yh[i] = __float2half_rn(__fadd_rn(__uint_as_float(r[i]), sm.shift[cc * 32 + i]));
      y[i]  = __half2float(yh[i]);
      wild  = wild || !(fabsf(y[i]) < tame_y);
    }
    if (Yout != nullptr) {
      uint4* dst = reinterpret_cast<uint4*>(Yout + static_cast<int64_t>(row) * N + c * 32);
#pragma unroll
      for (int i = 0; i < 4; i++)
        dst[i] = *reinterpret_cast<const uint4*>(&yh[8 * i]);
    }
    if (look.table == nullptr) {
      // codes of every level for a separate lookup kernel (and for inspection)
      long long* out = codes + (static_cast<int64_t>(row) * Cg + c) * L;
      for (int j = 0; j < L; j++) {
        long long h = 0;
        if (level_on == nullptr || level_on[c * L + j])
          h = wild ? cell_code<4>(y, sm.inv_f[j]) : cell_code_tame<4>(y, sm.inv_f[j]);
        out[j] = h;
      }
      continue;
    }
    // Lookup fused in (search_kernels.cuh:100-126: the finest level whose cell holds a list): the
    // table slot of a level is requested as soon as its code is known and looked at after the next
    // level has been decoded, so its latency hides behind that decode; once a level hits, the
    // coarser ones are not decoded at all. No code goes to memory.
    int2 sg         = make_int2(0, 0);
    bool found      = false, pending = false;
    int4 slot       = make_int4(0, 0, -1, 0);
    long long slot_h = 0;
    int slot_cl      = 0;
    long long tried = 0, scanned = 0;
    auto resolve = [&] {
      tried++;
      const unsigned mask = static_cast<unsigned>(look.tmask[slot_cl]);
      const cell_slot* tb = look.table + look.toff[slot_cl];
      unsigned s          = static_cast<unsigned>(slot_h) & mask;
      for (unsigned probe = 0; probe <= mask; probe++) {
        scanned++;
        if (slot.z < 0) break;  // an empty slot ends the run: no such cell
        const long long key = (static_cast<long long>(slot.y) << 32) | static_cast<unsigned>(slot.x);
        if (key == slot_h) {
          sg    = make_int2((look.base[slot_cl] + slot.z) * look.list_len, look.lr);
          found = true;
          break;
        }
        s    = (s + 1) & mask;
        slot = __ldg(reinterpret_cast<const int4*>(tb + s));
      }
      pending = false;
    };
    for (int j = 0; j < L && !found; j++) {
      const int cl = c * L + j;
      if (!level_on[cl]) continue;
      const long long h = wild ? cell_code<4>(y, sm.inv_f[j]) : cell_code_tame<4>(y, sm.inv_f[j]);
      if (pending) resolve();
      if (found) break;
      slot_h  = h;
      slot_cl = cl;
      slot    = __ldg(reinterpret_cast<const int4*>(look.table + look.toff[cl] +
                                                    (static_cast<unsigned>(h) & static_cast<unsigned>(look.tmask[cl]))));
      pending = true;
    }
    if (pending && !found) resolve();
    look.seg[static_cast<int64_t>(row) * Cg + c] = sg;
    if (look.stats != nullptr) {
      atomicAdd(reinterpret_cast<unsigned long long*>(look.stats + static_cast<int64_t>(row) * 8),
                static_cast<unsigned long long>(tried));
      atomicAdd(reinterpret_cast<unsigned long long*>(look.stats + static_cast<int64_t>(row) * 8 + 1),
                static_cast<unsigned long long>(scanned));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace

bool project_tc_supported(int blocks, int ldu) { return blocks == 4 && ldu % kTileK == 0; }

void project_tc_setup(project_tc_plan& p, const __half* qh, int m, const __half* ut, int copies, int ldu)
{
  p.m      = m;
  p.copies = copies;
  p.ldu    = ldu;
  make_map(p.map_a, qh, m, ldu, kTileM);
  make_map(p.map_b, ut, static_cast<int64_t>(copies) * 32, ldu, kTileN);
  cudaFuncSetAttribute(project_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(sizeof(tc_smem) + 1024));
}

void project_decode_tc(const project_tc_plan& p, int L, const __half* shift, const float* inv_f,
                       float finest, const unsigned char* level_on, long long* codes, __half* Yout,
                       const tc_lookup& look, int* error, cudaStream_t s)
{
  // |y| below this keeps |y / spacing| under the bound of the short decode at every level
  const float tame_y = finest > 0.f ? kTameLimit * finest * 0.99f : 0.f;
  if (p.m <= 0 || p.copies <= 0) return;
  CUtensorMap a, b;
  std::memcpy(&a, p.map_a, sizeof(a));
  std::memcpy(&b, p.map_b, sizeof(b));
  dim3 grid((p.copies * 32 + kTileN - 1) / kTileN, (p.m + kTileM - 1) / kTileM);
  project_decode_tc_kernel<<<grid, kThreads, sizeof(tc_smem) + 1024, s>>>(
    a, b, p.m, p.copies, L, p.ldu / kTileK, shift, inv_f, tame_y, level_on, codes, Yout, look, error);
}

}  // namespace octex_b200::kernels
