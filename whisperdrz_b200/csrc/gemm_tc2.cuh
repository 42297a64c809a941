// bf16 tensor-core GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias)
//
// Two CTAs of a cluster (an SM pair) share one 256x256 output tile.  Each CTA loads ITS 128 rows of A and ITS 128
// rows of W per 64-wide k-block (32 KB instead of the 48 KB a lone CTA needs for a 128x256 tile), the pair's leader
// issues one M256 N256 K16 MMA that reads both CTAs' shared memory, and each CTA ends up with its 128 rows of the
// accumulator in its own tensor memory.  One SM takes operands into shared memory at a fixed rate, and at 48 KB per
// k-block that rate, not the tensor pipe, bounds the lone-CTA kernel; the pair moves a third fewer bytes per flop.
//
//   warp 0      TMA producer in both CTAs (six 32 KB stages).  Loads carry .cta_group::2 so that their byte counts
//               complete on the LEADER's full barrier; the leader alone posts the expected 64 KB per stage.
//   warp 1      both CTAs allocate their 512 TMEM columns; the leader's lane 0 issues the MMAs and commits each
//               stage to the empty barrier of both CTAs, and the finished accumulator to both CTAs' acc_full.
//   warps 2-9   epilogue of the CTA's own 128 rows (same code as the lone-CTA kernel); every thread then arrives on
//               the leader's acc_empty barrier (512 arrivals), two accumulators alternate.
//
// Every mbarrier wait is bounded (status WDZ_ETIMEOUT, all roles leave); the two cluster barriers are reached by
// every thread of both CTAs after its bounded loops.
#pragma once
#include "gemm_tc.cuh"

namespace wdz {
namespace tc2 {

using tc::BK;
using tc::UMMA_K;
constexpr int BM_CTA = 128, BN = 256, BN_CTA = 128, PAIR_M = 256;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM_CTA * BK * 2, B_BYTES = BN_CTA * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
using tc::EPI_WARPS;
constexpr int THREADS = tc::THREADS;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;

// bf16 x bf16 -> f32, both operands K-major, M256 (the pair) x N256
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(PAIR_M >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(tc::smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads whose completion lands on a barrier of either CTA of the pair (bar: shared::cluster address)
__device__ __forceinline__ void tma_pair_load_3d(void* dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(tc::smem_u32(dst)), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_pair_load_2d(void* dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(tc::smem_u32(dst)), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
}
// arrive on one barrier (shared::cluster address, either CTA) when the pair's earlier MMAs have retired
__device__ __forceinline__ void umma_pair_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// grid = 2 x pairs (a multiple of two); p.tiles_m_per_batch counts 256-row pair tiles here
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const tc::TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                        // [STAGES]  used in the leader
  uint64_t* empty = bars + STAGES;              // [STAGES]  one set per CTA
  uint64_t* acc_full = bars + 2 * STAGES;       // [2]       one set per CTA
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]       used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { tc::mbar_init(full + i, 1); tc::mbar_init(empty + i, 1); }
    for (int i = 0; i < 2; ++i) { tc::mbar_init(acc_full + i, 1); tc::mbar_init(acc_empty + i, 2 * 32 * EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmW) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc::tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < p.total_tiles; tile += n_pairs) {
        const int nt = tile % p.tiles_n, mt_all = tile / p.tiles_n;
        const int b = mt_all / p.tiles_m_per_batch, mt = mt_all % p.tiles_m_per_batch;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int stage = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = tc::mbar_wait(empty + stage, phase ^ 1, abort_flag, p.status))) break;
          uint8_t* a_dst = smem + stage * STAGE_BYTES;
          if (leader) tc::mbar_expect_tx(full + stage, 2 * STAGE_BYTES);
          const uint32_t bar = map_to_cta(full + stage, 0);
          tma_pair_load_3d(a_dst, &tmA, bar, kb * BK, mt * PAIR_M + (int)rank * BM_CTA, b);
          tma_pair_load_2d(a_dst + A_BYTES, &tmW, bar, kb * BK, nt * BN + (int)rank * BN_CTA);
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      int it = 0, local = 0;
      bool ok = true;
      const uint32_t empty_leader = map_to_cta(empty, 0), empty_peer = map_to_cta(empty, 1);   // barriers are 8 bytes apart
      for (int tile = pair; ok && tile < p.total_tiles; tile += n_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!(ok = tc::mbar_wait(acc_empty + acc, acc_phase ^ 1, abort_flag, p.status))) break;
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int stage = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = tc::mbar_wait(full + stage, phase, abort_flag, p.status))) break;
          tc::tc_fence_after();
          const uint32_t a_addr = tc::smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = tc::umma_desc(a_addr), db = tc::umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_pair(d_tmem, da + (uint64_t)(k * (UMMA_K * 2 >> 4)), db + (uint64_t)(k * (UMMA_K * 2 >> 4)), (kb | k) != 0);
          umma_pair_commit(empty_leader + stage * 8);
          umma_pair_commit(empty_peer + stage * 8);
        }
        if (ok) {
          umma_pair_commit(map_to_cta(acc_full + acc, 0));
          umma_pair_commit(map_to_cta(acc_full + acc, 1));
        }
      }
    }
  } else {
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int c0 = ((warp - 2) >> 2) * (BN / 32 / (EPI_WARPS / 4));   // first 32-column chunk of this warp's share
    int local = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < p.total_tiles; tile += n_pairs, ++local) {
      const int nt = tile % p.tiles_n, mt_all = tile / p.tiles_n;
      const int b = mt_all / p.tiles_m_per_batch, mt = mt_all % p.tiles_m_per_batch;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = tc::mbar_wait(acc_full + acc, acc_phase, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective: leave together or not at all
      if (!ok) break;
      tc::tc_fence_after();
      const int t = mt * PAIR_M + (int)rank * BM_CTA + quad * 32 + lane;   // row inside the batch
      const int m = b * p.g.a_rpb + t;
      const bool row_ok = t < p.g.a_rpb && m < p.g.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      tc::epilogue_share<BN / 32 / (EPI_WARPS / 4)>(p.g, p.epi, row_ok, m, nt * BN + c0 * 32, taddr + c0 * 32);
      tc::tc_fence_before();
      mbar_arrive_cluster(map_to_cta(acc_empty + acc, 0));
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves (or frees TMEM) while the other may still read its memory or signal it
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

}  // namespace tc2
}  // namespace wdz
