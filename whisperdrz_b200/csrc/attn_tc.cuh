// Many-query attention on tcgen05 (head_dim 64, bf16 in, fp32 softmax):
// MultiHeadAttention.qkv_attention, src/whisperdrz/model.py:276-298.  Used for
// the encoder's self-attention (Q, K, V columns of one [B, T, 3d] tensor) and
// for the teacher-forced alignment pass of the decoder, where the queries of a
// chunk attend to its slot's cross cache, or causally to its self cache.
//
// One CTA per (128-query tile, head, window); two CTAs share an SM so that one
// CTA's softmax overlaps the other's MMAs.  Per 128-key tile:
//   S  = Q K^T        tcgen05.mma, both operands from 128-byte-swizzled shared
//                     memory (TMA), fp32 accumulator in TMEM columns [0,128)
//   P  = exp2(S*c - m) four softmax warps, one query row per thread: two passes
//                     of tcgen05.ld over S (row max, then exponentials), P
//                     packed to bf16 and written back to TMEM columns [128,192)
//                     with tcgen05.st
//   PV = P V          tcgen05.mma with the A operand read from TMEM and V used
//                     as an MN-major shared-memory operand (the [key][dim] tile
//                     exactly as TMA delivers it), result in columns [192,256)
// The running output stays in registers: O = (O + PV) * alpha, so no TMEM
// read-modify-write is needed.  K/V tiles are double-buffered.  Every mbarrier
// wait is bounded and reports WDZ_ETIMEOUT instead of hanging.
#pragma once
#include "attention.cuh"
#include "gemm_tc.cuh"

namespace wdz {
namespace atc {

using namespace tc;

constexpr int QT = 128, KT = 128, KV_STAGES = 2;
constexpr int TILE_BYTES = 128 * 128;           // 128 rows x 64 bf16
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KV_STAGES) + 256 + 1024;
constexpr int COL_S = 0, COL_P = 128, COL_O = 192, TMEM_COLS = 256;
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);

struct AttnTcParams {
  bf16* out;            // row (b * out_rows + q) holds query q of batch b, d columns
  int out_rows, d;
  int Tq, Tk;           // queries / keys per batch entry when no lengths are given
  const int* lens;      // optional [batches]: valid queries (and, if causal, keys) of a batch entry
  const int* kv_z;      // optional [batches]: third coordinate of the K / V maps (a cache slot); < 0 skips the batch
  int kv_z_base, kv_z_limit;   // added to kv_z[b] (layer * slots); slots
  int q_col0, k_col0, v_col0;  // first column of head 0 in the Q / K / V maps
  int causal;           // key k visible to query q only if k <= q
  int one_map;          // Q, K and V are columns of one tensor: only the first tensor map is fetched
  DevStatus* status;
};

__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// tcgen05.ld without the wait, so that two loads share one round trip.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
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
// Waits for the loads above; the registers pass through the statement so that no use can move ahead of it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&a)[32], uint32_t (&b)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(a[i]), "+r"(b[i]));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}

// kGeneral = false is the encoder's instantiation: no lengths, no slot indirection, no causal rule, one tensor
// map; those branches are then compiled out of its inner loops.
template <bool kGeneral>
__global__ void __launch_bounds__(192, 2)
attn_enc_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + TILE_BYTES;            // stage s: K at kv_s + s * 2 * TILE, V right after
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TILE_BYTES * (1 + 2 * KV_STAGES));
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                 // [2]
  uint64_t* kv_empty = bars + 3;                // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* s_empty = bars + 6;
  uint64_t* p_ready = bars + 7;
  uint64_t* pv_full = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * QT, h = blockIdx.y, b = blockIdx.z;
  // uniform over the CTA: nothing to do for tiles past the batch entry's queries or for skipped entries
  const int q_valid = (kGeneral && p.lens) ? min(p.lens[b], p.Tq) : p.Tq;
  const bool causal = kGeneral && p.causal;
  const bool one_map = !kGeneral || p.one_map;
  int kvz = b;
  if (kGeneral && p.kv_z) {
    const int z = p.kv_z[b];
    if (z < 0 || z >= p.kv_z_limit) return;
    kvz = p.kv_z_base + z;
  }
  if (q0 >= q_valid) {
    // padding queries: their output rows are zeroed so that later products of the pass stay finite
    // (a padded row's V would otherwise reach valid rows as 0 x NaN)
    const int rows = min(QT, p.Tq - q0);
    for (int i = threadIdx.x; i < rows * 8; i += blockDim.x)
      reinterpret_cast<uint4*>(p.out + ((int64_t)b * p.out_rows + q0 + (i >> 3)) * p.d + h * 64)[i & 7] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int k_valid = causal ? min(q_valid, p.Tk) : p.Tk;            // keys that exist
  const int k_end = causal ? min(k_valid, q0 + QT) : k_valid;        // keys this tile can see
  const int n_kv = (k_end + KT - 1) / KT;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) { mbar_init(kv_full + i, 1); mbar_init(kv_empty + i, 1); }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 128);
    mbar_init(p_ready, 128);
    mbar_init(pv_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmQ) : "memory");
    if (!one_map) {
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmK) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tmV) : "memory");
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      const CUtensorMap* mk = one_map ? &tmQ : &tmK;
      const CUtensorMap* mv = one_map ? &tmQ : &tmV;
      tma_load_3d(q_s, &tmQ, q_full, p.q_col0 + h * 64, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t phase = (j / KV_STAGES) & 1;
        if (!mbar_wait(kv_empty + st, phase ^ 1, abort_flag, p.status)) break;
        uint8_t* k_dst = kv_s + st * 2 * TILE_BYTES;
        mbar_expect_tx(kv_full + st, 2 * TILE_BYTES);
        tma_load_3d(k_dst, mk, kv_full + st, p.k_col0 + h * 64, j * KT, kvz);
        tma_load_3d(k_dst + TILE_BYTES, mv, kv_full + st, p.v_col0 + h * 64, j * KT, kvz);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status);
      const uint32_t q_addr = smem_u32(q_s);
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j % KV_STAGES;
        if (!(ok = mbar_wait(kv_full + st, (j / KV_STAGES) & 1, abort_flag, p.status))) break;
        if (!(ok = mbar_wait(s_empty, (j & 1) ^ 1, abort_flag, p.status))) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_s + st * 2 * TILE_BYTES);
        const uint32_t v_addr = k_addr + TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 4; ++k)   // contraction over the 64 head dims
          umma_idesc(tmem_base + COL_S, umma_desc(q_addr + k * 32), umma_desc(k_addr + k * 32), IDESC_S, k != 0);
        umma_commit(s_full);
        if (!(ok = mbar_wait(p_ready, j & 1, abort_flag, p.status))) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < KT / 16; ++k)  // contraction over the 128 keys; P holds two keys per TMEM column
          umma_ts(tmem_base + COL_O, tmem_base + COL_P + k * 8, umma_desc(v_addr + k * 2048), IDESC_PV, k != 0);
        umma_commit(pv_full);
        umma_commit(kv_empty + st);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    float m = -INFINITY, l = 0.0f, o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      ok = mbar_wait(s_full, j & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int k0 = j * KT;
      // only the last key tile has columns past the sequence; under the causal rule also the diagonal tile
      const bool tail = k0 + KT > k_valid || (causal && k0 + KT > q0);
      const int k_lim = causal ? min(k_valid, q + 1) : k_valid;   // keys [0, k_lim) are visible to this row
      float mx = -INFINITY;
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t a[32], b[32];
        tmem_ld32_issue(lane_addr + COL_S + hf * 64, a);
        tmem_ld32_issue(lane_addr + COL_S + hf * 64 + 32, b);
        tmem_ld_wait(a, b);
        if (!tail) {
          // four independent chains instead of one 64-long dependent chain
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            m0 = fmaxf(m0, __uint_as_float(a[i])); m1 = fmaxf(m1, __uint_as_float(a[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(b[i])); m3 = fmaxf(m3, __uint_as_float(b[i + 1]));
          }
          mx = fmaxf(mx, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (k0 + hf * 64 + i < k_lim) mx = fmaxf(mx, __uint_as_float(a[i]));
            if (k0 + hf * 64 + 32 + i < k_lim) mx = fmaxf(mx, __uint_as_float(b[i]));
          }
        }
      }
      const float m_new = fmaxf(m, mx * QK_SCALE_LOG2E);
      const float alpha = ex2(m - m_new);
      if (j > 0) {
        ok = mbar_wait(pv_full, (j - 1) & 1, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t a[32], b[32];
        tmem_ld32_issue(lane_addr + COL_O, a);
        tmem_ld32_issue(lane_addr + COL_O + 32, b);
        tmem_ld_wait(a, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          o[i] = (o[i] + __uint_as_float(a[i])) * alpha;
          o[32 + i] = (o[32 + i] + __uint_as_float(b[i])) * alpha;
        }
      }
      float sum = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t a[32], b[32], pk[32];
        tmem_ld32_issue(lane_addr + COL_S + hf * 64, a);
        tmem_ld32_issue(lane_addr + COL_S + hf * 64 + 32, b);
        tmem_ld_wait(a, b);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(fmaf(__uint_as_float(a[2 * i]), QK_SCALE_LOG2E, -m_new));
          float p1 = ex2(fmaf(__uint_as_float(a[2 * i + 1]), QK_SCALE_LOG2E, -m_new));
          float p2 = ex2(fmaf(__uint_as_float(b[2 * i]), QK_SCALE_LOG2E, -m_new));
          float p3 = ex2(fmaf(__uint_as_float(b[2 * i + 1]), QK_SCALE_LOG2E, -m_new));
          if (tail) {
            const int kk = k0 + hf * 64 + 2 * i;
            if (kk >= k_lim) p0 = 0.0f;
            if (kk + 1 >= k_lim) p1 = 0.0f;
            if (kk + 32 >= k_lim) p2 = 0.0f;
            if (kk + 33 >= k_lim) p3 = 0.0f;
          }
          sum += p0; sum1 += p1; sum2 += p2; sum3 += p3;
          pk[i] = pack_bf16(p0, p1);
          pk[16 + i] = pack_bf16(p2, p3);
        }
        tmem_st32(lane_addr + COL_P + hf * 32, pk);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      sum = (sum + sum1) + (sum2 + sum3);
      l = l * alpha + sum;
      m = m_new;
      tc_fence_before();
      mbar_arrive(s_empty);
      mbar_arrive(p_ready);
    }
    if (ok) {
      ok = mbar_wait(pv_full, (n_kv - 1) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      bf16* dst = p.out + ((int64_t)b * p.out_rows + q) * p.d + h * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld32(lane_addr + COL_O + c * 32, v);
        if (kGeneral && q >= q_valid && q < p.Tq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) reinterpret_cast<uint4*>(dst + c * 32)[g] = make_uint4(0, 0, 0, 0);
        }
        if (q < q_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 t;
            t.x = pack_bf16((o[c * 32 + 8 * g] + v[8 * g]) * inv, (o[c * 32 + 8 * g + 1] + v[8 * g + 1]) * inv);
            t.y = pack_bf16((o[c * 32 + 8 * g + 2] + v[8 * g + 2]) * inv, (o[c * 32 + 8 * g + 3] + v[8 * g + 3]) * inv);
            t.z = pack_bf16((o[c * 32 + 8 * g + 4] + v[8 * g + 4]) * inv, (o[c * 32 + 8 * g + 5] + v[8 * g + 5]) * inv);
            t.w = pack_bf16((o[c * 32 + 8 * g + 6] + v[8 * g + 6]) * inv, (o[c * 32 + 8 * g + 7] + v[8 * g + 7]) * inv);
            reinterpret_cast<uint4*>(dst + c * 32)[g] = t;
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace atc
}  // namespace wdz
