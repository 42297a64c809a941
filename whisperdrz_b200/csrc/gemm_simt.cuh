// CUDA-core GEMMs: C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias).
//
// Two shapes of the same product:
//   gemm_tile_kernel  - 64x64x16 shared-memory tiles, fp32 FMA.  It is the
//                       arithmetic of the fp32 mode (no tensor cores, so that
//                       greedy tokens match the fp32 reference) and the
//                       correctness fallback of the bf16 mode.
//   gemv_rows_kernel  - M <= a few dozen rows (decode): each warp streams whole
//                       rows of W once with 16-byte loads and keeps an 8-row
//                       register tile of outputs; HBM-bound on the weights.
// Both operands are K-major, exactly as nn.Linear stores them
// (y = x W^T + b, src/whisperdrz/model.py:258-261,387-393).
#pragma once
#include "common.cuh"

namespace wdz {

enum Epi : int {
  EPI_STORE = 0,     // C = acc + bias
  EPI_GELU = 1,      // C = gelu(acc + bias)
  EPI_RESID = 2,     // C(f32) += acc + bias            (residual stream update)
  EPI_GELU_POS = 3,  // C(f32) = gelu(acc + bias) + pos[m % rows_per_batch, n]   (conv2 + positional add)
  EPI_CROSS_KV = 4,  // scatter columns (layer, k|v, channel) and rows (window, t) into the slotted caches
};

struct GemmParams {
  const void* A; const void* W; const void* bias; void* C;
  int M, N, K;
  int64_t lda, ldc;
  // A row m lives at A + (m / a_rpb) * a_bstride + (m % a_rpb) * lda; same for C with c_*.
  int a_rpb; int64_t a_bstride;
  int c_rpb; int64_t c_bstride;
  const float* pos;          // EPI_GELU_POS: [a_rpb, N]
  // EPI_CROSS_KV
  void* cache_k; void* cache_v; const int* slot_ids; int n_slots, T, d;
};

template <typename TW, typename TO>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, int epi, int m, int n, float acc) {
  if (p.bias) acc += to_f(reinterpret_cast<const TW*>(p.bias)[n]);
  if (epi == EPI_CROSS_KV) {
    const int layer = n / (2 * p.d), kv = (n / p.d) & 1, c = n % p.d;
    const int w = m / p.T, t = m % p.T;
    const int slot = p.slot_ids[w];
    TO* dst = reinterpret_cast<TO*>(kv ? p.cache_v : p.cache_k);
    dst[(((int64_t)layer * p.n_slots + slot) * p.T + t) * p.d + c] = from_f<TO>(acc);
    return;
  }
  const int64_t off = (int64_t)(m / p.c_rpb) * p.c_bstride + (int64_t)(m % p.c_rpb) * p.ldc + n;
  if (epi == EPI_STORE) {
    reinterpret_cast<TO*>(p.C)[off] = from_f<TO>(acc);
  } else if (epi == EPI_GELU) {
    reinterpret_cast<TO*>(p.C)[off] = from_f<TO>(gelu_erf(acc));
  } else if (epi == EPI_RESID) {
    reinterpret_cast<float*>(p.C)[off] += acc;
  } else {  // EPI_GELU_POS
    reinterpret_cast<float*>(p.C)[off] = gelu_erf(acc) + p.pos[(int64_t)(m % p.a_rpb) * p.N + n];
  }
}

// bias is stored in the weight type TW; outputs of EPI_STORE / EPI_GELU / EPI_CROSS_KV in TO.
template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256) gemm_tile_kernel(GemmParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int BM = 64, BN = 64, BK = 16, LD = 68;
  __shared__ float As[BK][LD];
  __shared__ float Ws[BK][LD];
  const TA* A = reinterpret_cast<const TA*>(p.A);
  const TW* W = reinterpret_cast<const TW*>(p.W);
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row 0..63, k offset 0/4/8/12

  const int am = m0 + lr;
  const TA* a_row = nullptr;
  if (am < p.M) a_row = A + (int64_t)(am / p.a_rpb) * p.a_bstride + (int64_t)(am % p.a_rpb) * p.lda;
  const int wn = n0 + lr;
  const TW* w_row = wn < p.N ? W + (int64_t)wn * p.K : nullptr;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lr] = a_row ? to_f(a_row[k0 + lk + i]) : 0.0f;
      Ws[lk + i][lr] = w_row ? to_f(w_row[k0 + lk + i]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 16 * i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n < p.N) epilogue_store<TW, TO>(p, EPI, m, n, acc[i][j]);
    }
  }
}

// Decode-shaped product: x f32 [M, K] (rows gathered through row_idx when not
// NULL), W TW [N, K], y f32.  One warp owns CPW output columns and walks the
// M rows eight at a time; lanes split K in 16-byte pieces of W.
struct GemvParams {
  const float* x; const void* W; const void* bias; float* y;
  int M, N, K;
  int64_t ldx, ldy;
  const int* row_idx;
};

template <typename TW, int EPI, int CPW>
__global__ void __launch_bounds__(256) gemv_rows_kernel(GemvParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int VEC = Vec<TW>::N;
  constexpr int MT = 8;
  const TW* W = reinterpret_cast<const TW*>(p.W);
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * 256 + threadIdx.x) >> 5;
  const int n0 = warp * CPW;
  if (n0 >= p.N) return;
  const int nvec = p.K / VEC;

  for (int mb = 0; mb < p.M; mb += MT) {
    float acc[CPW][MT];
#pragma unroll
    for (int c = 0; c < CPW; ++c)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[c][m] = 0.0f;
    const float* xr[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int r = mb + m < p.M ? mb + m : p.M - 1;
      if (p.row_idx) r = p.row_idx[r];
      xr[m] = p.x + (int64_t)r * p.ldx;
    }
    for (int v = lane; v < nvec; v += 32) {
      float w[CPW][VEC];
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const int n = n0 + c < p.N ? n0 + c : p.N - 1;
        load_vec_nc(W + (int64_t)n * p.K + (int64_t)v * VEC, w[c]);
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float xv[VEC];
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          const float4 t = *reinterpret_cast<const float4*>(xr[m] + (int64_t)v * VEC + 4 * q);
          xv[4 * q] = t.x; xv[4 * q + 1] = t.y; xv[4 * q + 2] = t.z; xv[4 * q + 3] = t.w;
        }
#pragma unroll
        for (int c = 0; c < CPW; ++c)
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[c][m] = fmaf(w[c][e], xv[e], acc[c][m]);
      }
    }
#pragma unroll
    for (int c = 0; c < CPW; ++c)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[c][m] = warp_sum(acc[c][m]);
    if (lane < MT && mb + lane < p.M) {
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const int n = n0 + c;
        if (n >= p.N) continue;
        float v = 0.0f;
#pragma unroll
        for (int m = 0; m < MT; ++m) v = lane == m ? acc[c][m] : v;
        if (p.bias) v += to_f(reinterpret_cast<const TW*>(p.bias)[n]);
        float* dst = p.y + (int64_t)(mb + lane) * p.ldy + n;
        if (EPI == EPI_STORE) *dst = v;
        else if (EPI == EPI_GELU) *dst = gelu_erf(v);
        else *dst += v;  // EPI_RESID
      }
    }
  }
}

}  // namespace wdz
