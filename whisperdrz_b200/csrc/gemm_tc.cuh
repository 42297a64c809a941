// bf16 tensor-core GEMM for sm_100a: C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias)
// with TMA-fed shared-memory tiles, tcgen05.mma accumulating in tensor memory
// and a warp-specialised, persistent schedule:
//
//   warp 0      TMA producer: 128x64 tile of A and 256x64 tile of W per stage
//               (128-byte swizzle), four stages, mbarrier full/empty pairs
//   warp 1      allocates the 512 TMEM columns and issues tcgen05.mma
//               (M128 N256 K16, four per stage); tcgen05.commit releases the
//               stage and, after the last k-block, publishes the accumulator
//   warps 2-9   epilogue: tcgen05.ld of their 32-lane TMEM quadrant (two warps
//               per quadrant, 128 columns each), bias / GELU / residual /
//               positional add / KV-cache scatter, 16-byte global stores.  Two
//               256-column accumulators alternate so the epilogue of tile i
//               overlaps the main loop of tile i+1.  Eight warps because the
//               exact-erf GELU is bound by instruction issue: with four, one per
//               scheduler, the fc1 epilogue took longer than its main loop.
//
// The grid is one CTA per SM; tiles are taken round-robin with the N index
// fastest so that CTAs running together share their A rows through L2.
// A is addressed through a 3-D tensor map (k, row-in-batch, batch) so that the
// stride-2 convolution can read overlapping 3-row windows of its input with
// no im2col copy; rows past the end of a batch are zero-filled by TMA.
//
// Every mbarrier wait is bounded: when it runs out the kernel records
// WDZ_ETIMEOUT in the engine's status word and all roles leave their loops.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "gemm_simt.cuh"

namespace wdz {
namespace tc {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;                 // two per TMEM lane quadrant, each takes half of a tile's columns
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;  // tiles + barriers + alignment slack
constexpr long long WAIT_CYCLES = 2000000000ll;                // ~1 s

struct TcParams {
  GemmParams g;
  int epi;
  int tiles_m_per_batch, batches, tiles_n, total_tiles, kblocks;
  DevStatus* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, DevStatus* status) {
  const uint32_t a = smem_u32(bar);
  const long long t0 = clock64();
  for (int spin = 0;; ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
    if ((spin & 63) == 63) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_CYCLES) {
        *abort_flag = 1;
        if (status) { atomicCAS(&status->code, 0, WDZ_ETIMEOUT); status->detail = (int)blockIdx.x; }
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte
// swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);       // start address
  d |= (uint64_t)0 << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset
  d |= (uint64_t)1 << 46;                            // descriptor version
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M128 x N256.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait, and the wait with the registers threaded through it, so that a
// second load can be in flight while the first one's values are used.
__device__ __forceinline__ void tmem_ld32_raw(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(r[i]));
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// One row m, 32 consecutive columns starting at n (n % 32 == 0).
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, int epi, int m, int n, float (&v)[32]) {
  if (p.bias) {
    const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.bias) + n);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 t = __ldg(bp + q);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[8 * q + 2 * i] += __uint_as_float(w[i] << 16);
        v[8 * q + 2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  }
  if (epi == EPI_STORE || epi == EPI_GELU || epi == EPI_CROSS_KV) {
    bf16* dst;
    if (epi == EPI_CROSS_KV) {
      const int layer = n / (2 * p.d), kv = (n / p.d) & 1, c = n % p.d;
      const int w = m / p.T, t = m % p.T;
      const int slot = p.slot_ids[w];
      dst = reinterpret_cast<bf16*>(kv ? p.cache_v : p.cache_k) +
            (((int64_t)layer * p.n_slots + slot) * p.T + t) * p.d + c;
    } else {
      dst = reinterpret_cast<bf16*>(p.C) + (int64_t)(m / p.c_rpb) * p.c_bstride + (int64_t)(m % p.c_rpb) * p.ldc + n;
    }
    if (epi == EPI_GELU) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_fast(v[i]);
    }
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 t;
      t.x = pack_bf16(v[8 * q], v[8 * q + 1]);
      t.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
      t.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]);
      t.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
      d4[q] = t;
    }
  } else {
    float4* d4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + (int64_t)(m / p.c_rpb) * p.c_bstride +
                                           (int64_t)(m % p.c_rpb) * p.ldc + n);
    if (epi == EPI_RESID) {
      // one addend per element (K is not split here), so a fire-and-forget reduction gives the same fp32 sum as
      // load-add-store - without the epilogue warps waiting a memory latency per 32 columns
#pragma unroll
      for (int q = 0; q < 8; ++q)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(d4 + q), "f"(v[4 * q]), "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
    } else {  // EPI_GELU_POS
      const float4* pp = reinterpret_cast<const float4*>(p.pos + (int64_t)(m % p.a_rpb) * p.N + n);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 ps = __ldg(pp + q);
        float4 t;
        t.x = gelu_fast(v[4 * q]) + ps.x; t.y = gelu_fast(v[4 * q + 1]) + ps.y;
        t.z = gelu_fast(v[4 * q + 2]) + ps.z; t.w = gelu_fast(v[4 * q + 3]) + ps.w;
        d4[q] = t;
      }
    }
  }
}

// One epilogue warp's share of a tile: NCH chunks of 32 columns from TMEM address taddr, first column n0.  The TMEM
// load of the next chunk is in flight while the current one goes through bias / activation / stores.
template <int NCH>
__device__ __forceinline__ void epilogue_share(const GemmParams& g, int epi, bool row_ok, int m, int n0, uint32_t taddr) {
  static_assert(NCH % 2 == 0, "chunks are taken in pairs");
  uint32_t ra[32], rb[32];
  float v[32];
  tmem_ld32_raw(taddr, ra);
#pragma unroll 1
  for (int c = 0; c < NCH; c += 2) {
    tmem_wait_ld(ra);
    tmem_ld32_raw(taddr + (c + 1) * 32, rb);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
    if (row_ok) epilogue_chunk(g, epi, m, n0 + c * 32, v);
    tmem_wait_ld(rb);
    if (c + 2 < NCH) tmem_ld32_raw(taddr + (c + 2) * 32, ra);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rb[i]);
    if (row_ok) epilogue_chunk(g, epi, m, n0 + (c + 1) * 32, v);
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                 // [STAGES]
  uint64_t* empty = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;   // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 32 * EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmW) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        const int nt = tile % p.tiles_n, mt_all = tile / p.tiles_n;
        const int b = mt_all / p.tiles_m_per_batch, mt = mt_all % p.tiles_m_per_batch;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int stage = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, p.status))) break;
          uint8_t* a_dst = smem + stage * STAGE_BYTES;
          mbar_expect_tx(full + stage, STAGE_BYTES);
          tma_load_3d(a_dst, &tmA, full + stage, kb * BK, mt * BM, b);
          tma_load_2d(a_dst + A_BYTES, &tmW, full + stage, kb * BK, nt * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!(ok = mbar_wait(acc_empty + acc, acc_phase ^ 1, abort_flag, p.status))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int stage = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(full + stage, phase, abort_flag, p.status))) break;
          tc_fence_after();
          // descriptors once per stage; the next 16 columns of k are 32 bytes on = +2 in the address field (the
          // issuing thread shares its scheduler with two epilogue warps, every instruction here is paid in MMA gaps)
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(d_tmem, da + (uint64_t)(k * (UMMA_K * 2 >> 4)), db + (uint64_t)(k * (UMMA_K * 2 >> 4)), (kb | k) != 0);
          umma_commit(empty + stage);
        }
        if (ok) umma_commit(acc_full + acc);
      }
    }
  } else {
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int c0 = ((warp - 2) >> 2) * (BN / 32 / (EPI_WARPS / 4));   // first 32-column chunk of this warp's share
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++local) {
      const int nt = tile % p.tiles_n, mt_all = tile / p.tiles_n;
      const int b = mt_all / p.tiles_m_per_batch, mt = mt_all % p.tiles_m_per_batch;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(acc_full + acc, acc_phase, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective: leave together or not at all
      if (!ok) break;
      tc_fence_after();
      const int t = mt * BM + quad * 32 + lane;       // row inside the batch
      const int m = b * p.g.a_rpb + t;
      const bool row_ok = t < p.g.a_rpb && m < p.g.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      epilogue_share<BN / 32 / (EPI_WARPS / 4)>(p.g, p.epi, row_ok, m, nt * BN + c0 * 32, taddr + c0 * 32);
      tc_fence_before();
      mbar_arrive(acc_empty + acc);
    }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Decode-shaped product on tcgen05 with the operands swapped:
//   D[feature, row] = W[128-feature tile, K] . x[row tile, K]^T
// so that the 128-wide MMA M dimension is filled by output features and a
// tile of 32 to 256 token rows forms the MMA N dimension.  W comes from HBM
// once per call (row tiles of the same features run together and share it
// through L2).  grid = (feature tiles, K splits, row tiles): the host picks
// the row tile and the K split so that the CTAs cover the SMs - a call is
// bounded by the rate at which one SM takes operand bytes into shared memory
// (about 0.3-0.4 us per 64-wide k-block), not by the weight stream.  With
// more than one K split the partial sums are added to the fp32 output with
// red.global.add (residual-stream epilogue only).
// Epilogue thread = one feature (TMEM lane), columns = rows; eight epilogue
// warps, two per lane quadrant, each taking half of the row tile.
// ---------------------------------------------------------------------------
constexpr int SW_STAGES = 4;
constexpr int SW_THREADS = 320;   // producer warp, MMA warp, eight epilogue warps (two per TMEM lane quadrant)
constexpr int SW_STAGE_BYTES = A_BYTES + 256 * BK * 2;   // W tile + up to 256 rows of x
constexpr int SW_SMEM_BYTES = SW_STAGES * SW_STAGE_BYTES + 256 + 1024;   // largest launch
inline int sw_smem_bytes(int row_tile) { return SW_STAGES * (A_BYTES + row_tile * BK * 2) + 256 + 1024; }
constexpr int EPI_SW_QKV_CACHE = 16;

struct TcSwapParams {
  const bf16* bias; void* y; int64_t ldy;
  int M, N, K;               // rows, features, contraction
  int mpad;                  // rows of one CTA's row tile, a multiple of 32 (MMA N)
  int tmem_cols;             // power of two >= mpad, >= 32
  int kb_per_split, kblocks;
  int epi;                   // EPI_STORE (f32) | EPI_GELU (bf16 out) | EPI_RESID (f32 +=) | EPI_SW_QKV_CACHE
  uint32_t idesc;
  bf16* cache_k; bf16* cache_v; const int* slots; const int* positions;
  int layer, n_slots, S, d;
  DevStatus* status;
};

__device__ __forceinline__ void umma_idesc(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(SW_THREADS, 1)
gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const TcSwapParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t w_bytes = A_BYTES;                               // 128 features x 64 k, 16 KB
  const uint32_t stage_bytes = w_bytes + (uint32_t)p.mpad * BK * 2;   // a multiple of 1024
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SW_STAGES * stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + SW_STAGES;
  uint64_t* acc_full = bars + 2 * SW_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SW_STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x;
  const int row0 = blockIdx.z * p.mpad;           // first token row of this CTA's row tile
  const int kb0 = blockIdx.y * p.kb_per_split;
  const int kb1 = min(p.kblocks, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;   // >= 1 by construction of the grid
  if (threadIdx.x == 0) {
    for (int i = 0; i < SW_STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmW) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmX) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_trigger();
  pdl_wait();   // barriers, TMEM and tensor-map prefetch above overlap the previous kernel
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int stage = i % SW_STAGES;
        const uint32_t phase = (i / SW_STAGES) & 1;
        if (!mbar_wait(empty + stage, phase ^ 1, abort_flag, p.status)) break;
        uint8_t* w_dst = smem + stage * stage_bytes;
        mbar_expect_tx(full + stage, stage_bytes);
        tma_load_2d(w_dst, &tmW, full + stage, (kb0 + i) * BK, tile * BM);
        tma_load_2d(w_dst + w_bytes, &tmX, full + stage, (kb0 + i) * BK, row0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int stage = i % SW_STAGES;
        const uint32_t phase = (i / SW_STAGES) & 1;
        if (!(ok = mbar_wait(full + stage, phase, abort_flag, p.status))) break;
        tc_fence_after();
        const uint32_t w_addr = smem_u32(smem + stage * stage_bytes);
        const uint64_t dw = umma_desc(w_addr), dx = umma_desc(w_addr + w_bytes);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_idesc(tmem_base, dw + (uint64_t)(k * (UMMA_K * 2 >> 4)), dx + (uint64_t)(k * (UMMA_K * 2 >> 4)), p.idesc, (i | k) != 0);
        umma_commit(empty + stage);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quad = warp & 3;
    bool ok = mbar_wait(acc_full, 0, abort_flag, p.status);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      // MMA M = 128: accumulator row r (a feature) sits in TMEM lane r
      const int n = tile * BM + quad * 32 + lane;   // output feature of this thread
      const bool n_ok = n < p.N;
      float bias = 0.0f;
      if (n_ok && p.bias && blockIdx.y == 0) bias = to_f(p.bias[n]);
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
      // 32 rows per TMEM load; the load of the next 32 rows is in flight while these are written out
      auto emit = [&](int c, const uint32_t (&r)[32]) {   // c: first token row of the 32 in r
        if (!n_ok) return;
        const int rows = min(32, p.M - c);
        if (p.epi == EPI_RESID) {
          float* dst = reinterpret_cast<float*>(p.y) + (int64_t)c * p.ldy + n;
          // fire-and-forget adds, also without a K split (one addend per element then: the same fp32 sum as
          // load-add-store, without the loads' latency)
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < rows) atomicAdd(dst + (int64_t)j * p.ldy, __uint_as_float(r[j]) + bias);
        } else if (p.epi == EPI_GELU) {
          bf16* dst = reinterpret_cast<bf16*>(p.y) + (int64_t)c * p.ldy + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < rows) dst[(int64_t)j * p.ldy] = from_f<bf16>(gelu_fast(__uint_as_float(r[j]) + bias));
        } else if (p.epi == EPI_SW_QKV_CACHE && n >= p.d) {
          const bool is_v = n >= 2 * p.d;
          bf16* cache = is_v ? p.cache_v : p.cache_k;
          const int col = n - (is_v ? 2 : 1) * p.d;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < rows) {
              const int sl = p.slots[c + j], pos = p.positions[c + j];
              if (sl >= 0 && sl < p.n_slots && pos >= 0 && pos < p.S)
                cache[(((int64_t)p.layer * p.n_slots + sl) * p.S + pos) * p.d + col] =
                    from_f<bf16>(__uint_as_float(r[j]) + bias);
            }
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.y) + (int64_t)c * p.ldy + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < rows) dst[(int64_t)j * p.ldy] = __uint_as_float(r[j]) + bias;
        }
      };
      // the two warps of a lane quadrant split the row tile's 32-row groups: the epilogue runs after the main loop
      // (one tile per CTA), so its length is paid in full on every product
      const int groups = p.mpad >> 5, mid = (groups + 1) >> 1;
      const int c_lo = ((warp - 2) >> 2) ? mid * 32 : 0, c_hi = ((warp - 2) >> 2) ? groups * 32 : mid * 32;
      uint32_t ra[32], rb[32];
      if (c_lo < c_hi) tmem_ld32_raw(taddr + c_lo, ra);
      for (int c = c_lo; c < c_hi; c += 64) {
        tmem_wait_ld(ra);
        if (c + 32 < c_hi) tmem_ld32_raw(taddr + c + 32, rb);
        if (row0 + c < p.M) emit(row0 + c, ra);
        if (c + 32 < c_hi) {
          tmem_wait_ld(rb);
          if (c + 64 < c_hi) tmem_ld32_raw(taddr + c + 64, ra);
          if (row0 + c + 32 < p.M) emit(row0 + c + 32, rb);
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn& encode_fn() {
  static EncodeTiledFn fn = nullptr;
  return fn;
}

// bf16 tensor [d2][d1][d0] with byte strides s1, s2 (d0 contiguous); box = {64, box1, 1}.
inline bool make_map(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                     uint64_t s2, uint32_t box1, int rank) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {(cuuint32_t)BK, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace wdz
