// Decode-shaped bf16 product on the tensor cores: y[M, N] = epi(x[M, K] . W[N, K]^T + bias)
// for M up to a few hundred token rows.  The product is HBM-bound on W
// (every weight is read once per step), so the kernel is built around the
// weight stream, not around the MMA:
//
//   - a CTA owns 16 output features; its 8 warps split K eight ways and each
//     streams its slice of the 16 weight rows straight from global memory
//     into MMA A-fragments with 16-byte loads (no shared-memory staging);
//   - x (bf16, L2-resident, a few hundred KB) is read as the B fragment with
//     the same 16-byte pattern;
//   - mma.sync.m16n8k16 (features x rows) accumulates in fp32; the eight
//     K-slices are summed through shared memory and the epilogue (bias, GELU,
//     residual add, or the Q / K-cache / V-cache split of the fused QKV
//     projection) runs on the complete sums - no atomics, deterministic.
//
// Within each 32-wide k block a lane loads 8 consecutive k of one row; the
// two MMAs of the block take elements {0..3} and {4..7} of every lane.  The
// k index inside an MMA is only a label, and A and B use the same labelling,
// so the contraction is exact.
#pragma once
#include "common.cuh"
#include "gemm_simt.cuh"

namespace wdz {

struct GemvMmaParams {
  const bf16* x; int64_t ldx;
  const bf16* W; const bf16* bias;
  void* y; int64_t ldy;      // f32, or bf16 when OUT_BF16
  int M, N, K;
  // EPI_QKV_CACHE: columns [0, d) -> y (queries, f32 [M, d]); [d, 2d) and [2d, 3d) -> K / V cache rows
  bf16* cache_k; bf16* cache_v; const int* slots; const int* positions;
  int layer, n_slots, S, d;
  // weights of the product that runs next: pulled into L2 while this one streams its own
  const void* next_w; size_t next_bytes;
};

// Each CTA asks L2 for its share of [ptr, ptr + bytes) in 128-byte lines.
__device__ __forceinline__ void l2_prefetch_share(const void* ptr, size_t bytes, int cta, int n_cta, int tid, int n_thr) {
  if (!ptr || bytes == 0) return;
  const size_t lines = (bytes + 127) >> 7;
  const size_t per = (lines + n_cta - 1) / n_cta;
  const size_t lo = per * cta, hi = lo + per < lines ? lo + per : lines;
  const char* base = reinterpret_cast<const char*>(ptr);
  for (size_t i = lo + tid; i < hi; i += n_thr)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (i << 7)));
}

constexpr int EPI_QKV_CACHE = 16;
constexpr int GEMV_MMA_MAXROWS = 16;  // rows per pass (2 MMA n-tiles): keeps registers low, several CTAs per SM
constexpr int GEMV_MMA_TILES = GEMV_MMA_MAXROWS / 8;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int EPI, bool OUT_BF16>
__global__ void __launch_bounds__(256, 4) gemv_mma_kernel(GemvMmaParams p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8][16][GEMV_MMA_MAXROWS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int kslice = p.K >> 3;                       // K % 256 == 0
  const int kbeg = warp * kslice;
  const int ra = min(n0 + g, p.N - 1), rb = min(n0 + g + 8, p.N - 1);
  const bf16* wa_ptr = p.W + (int64_t)ra * p.K + kbeg + 8 * q;
  const bf16* wb_ptr = p.W + (int64_t)rb * p.K + kbeg + 8 * q;
  l2_prefetch_share(p.next_w, p.next_bytes, blockIdx.x, gridDim.x, threadIdx.x, 256);

  for (int m0 = 0; m0 < p.M; m0 += GEMV_MMA_MAXROWS) {
    const int rows = min(GEMV_MMA_MAXROWS, p.M - m0);
    const int tiles = (rows + 7) >> 3;
    float acc[GEMV_MMA_TILES][4];
#pragma unroll
    for (int t = 0; t < GEMV_MMA_TILES; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] = 0.0f;
    const bf16* xrow[GEMV_MMA_TILES];
#pragma unroll
    for (int t = 0; t < GEMV_MMA_TILES; ++t) xrow[t] = p.x + (int64_t)min(m0 + t * 8 + g, p.M - 1) * p.ldx + kbeg + 8 * q;

#pragma unroll 5
    for (int kb = 0; kb < kslice; kb += 32) {
      const uint4 wa = __ldg(reinterpret_cast<const uint4*>(wa_ptr + kb));
      const uint4 wb = __ldg(reinterpret_cast<const uint4*>(wb_ptr + kb));
#pragma unroll
      for (int t = 0; t < GEMV_MMA_TILES; ++t) {
        if (t < tiles) {
          const uint4 xb = *reinterpret_cast<const uint4*>(xrow[t] + kb);
          mma_bf16_16816(acc[t], wa.x, wb.x, wa.y, wb.y, xb.x, xb.y);
          mma_bf16_16816(acc[t], wa.z, wb.z, wa.w, wb.w, xb.z, xb.w);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < GEMV_MMA_TILES; ++t) {
      if (t < tiles) {
        red[warp][g][t * 8 + 2 * q] = acc[t][0];
        red[warp][g][t * 8 + 2 * q + 1] = acc[t][1];
        red[warp][g + 8][t * 8 + 2 * q] = acc[t][2];
        red[warp][g + 8][t * 8 + 2 * q + 1] = acc[t][3];
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * rows; i += 256) {
      const int f = i & 15, mm = i >> 4;
      const int n = n0 + f, m = m0 + mm;
      if (n >= p.N) continue;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w) v += red[w][f][mm];
      if (p.bias) v += to_f(p.bias[n]);
      if (EPI == EPI_QKV_CACHE) {
        if (n < p.d) {
          reinterpret_cast<float*>(p.y)[(int64_t)m * p.ldy + n] = v;
        } else {
          const int s = p.slots[m], pos = p.positions[m];
          if (s >= 0 && s < p.n_slots && pos >= 0 && pos < p.S) {
            const bool is_v = n >= 2 * p.d;
            bf16* dst = is_v ? p.cache_v : p.cache_k;
            dst[(((int64_t)p.layer * p.n_slots + s) * p.S + pos) * p.d + (n - (is_v ? 2 : 1) * p.d)] = from_f<bf16>(v);
          }
        }
      } else {
        if (EPI == EPI_GELU) v = gelu_erf(v);
        if (OUT_BF16) {
          reinterpret_cast<bf16*>(p.y)[(int64_t)m * p.ldy + n] = from_f<bf16>(v);
        } else {
          float* dst = reinterpret_cast<float*>(p.y) + (int64_t)m * p.ldy + n;
          if (EPI == EPI_RESID) *dst += v; else *dst = v;
        }
      }
    }
    __syncthreads();
  }
}

}  // namespace wdz
