// Row-wise helpers around the GEMMs: LayerNorm over the fp32 residual stream
// (src/whisperdrz/model.py:195-200, eps 1e-5), token + learned positional
// embedding (model.py:597), the conv1 im2col (model.py:449,467), K/V append
// into the slotted self-attention cache (model.py:51-54) and slot bookkeeping.
#pragma once
#include "common.cuh"

namespace wdz {

// y[r] = LN(x[src(r)]) * gamma + beta.  One warp per row; the row is read
// once with 16-byte loads that are all issued before the first use (rows of
// up to 2048 elements live in registers), then mean, centred variance and the
// affine output are computed from the registers.  d % 4 == 0, d <= 2048.
template <typename TP, typename TO>
__global__ void __launch_bounds__(128)
layernorm_kernel(const float* __restrict__ x, int64_t ldx, const int* __restrict__ row_idx,
                 const TP* __restrict__ gamma, const TP* __restrict__ beta,
                 TO* __restrict__ y, int64_t ldy, int rows, int d) {
  pdl_trigger();
  pdl_wait();
  constexpr int MAXV = 16;  // float4 per lane
  const int r = (blockIdx.x * 128 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)(row_idx ? row_idx[r] : r) * ldx);
  const int nv = d >> 2;
  float4 v[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int j = lane + 32 * i;
    v[i] = j < nv ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  const float mean = warp_sum(s) / d;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if (lane + 32 * i < nv) {
      const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      q += a * a + b * b + c * c + e * e;
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / d + 1e-5f);
  TO* yr = y + (int64_t)r * ldy;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int j = lane + 32 * i;
    if (j < nv) {
      const int c = 4 * j;
      yr[c] = from_f<TO>((v[i].x - mean) * rstd * to_f(gamma[c]) + to_f(beta[c]));
      yr[c + 1] = from_f<TO>((v[i].y - mean) * rstd * to_f(gamma[c + 1]) + to_f(beta[c + 1]));
      yr[c + 2] = from_f<TO>((v[i].z - mean) * rstd * to_f(gamma[c + 2]) + to_f(beta[c + 2]));
      yr[c + 3] = from_f<TO>((v[i].w - mean) * rstd * to_f(gamma[c + 3]) + to_f(beta[c + 3]));
    }
  }
}

// x[r] = E[token[r]] + P[position[r]]  (fp32 residual stream).
template <typename TP>
__global__ void __launch_bounds__(256)
embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
             const TP* __restrict__ E, const TP* __restrict__ P, float* __restrict__ x,
             int rows, int d, int n_vocab, int n_ctx) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  int t = tokens[r], pos = positions[r];
  t = t < 0 ? 0 : (t >= n_vocab ? n_vocab - 1 : t);
  pos = pos < 0 ? 0 : (pos >= n_ctx ? n_ctx - 1 : pos);
  for (int i = threadIdx.x; i < d; i += 256)
    x[(int64_t)r * d + i] = to_f(E[(int64_t)t * d + i]) + to_f(P[(int64_t)pos * d + i]);
}

// positions[r] = seq_lens[slot[r]]  (decode step: the next free position of each slot).
__global__ void positions_from_seqlens_kernel(const int* __restrict__ slots, const int* __restrict__ seq_lens,
                                              int* __restrict__ positions, int n, int n_slots) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int s = slots[r];
  positions[r] = (s >= 0 && s < n_slots) ? seq_lens[s] : 0;
}

// seq_lens[slot[r]] = max(seq_lens[slot[r]], position[r] + 1)
__global__ void bump_seqlens_kernel(const int* __restrict__ slots, const int* __restrict__ positions,
                                    int* __restrict__ seq_lens, int n, int n_slots) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int s = slots[r];
  if (s >= 0 && s < n_slots) atomicMax(seq_lens + s, positions[r] + 1);
}

__global__ void reset_seqlens_kernel(const int* __restrict__ slots, int* __restrict__ seq_lens, int n, int n_slots) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int s = slots[r];
  if (s >= 0 && s < n_slots) seq_lens[s] = 0;
}

// cache[layer][slot][pos][:] = qkv[r][d + :] (K) and qkv[r][2d + :] (V).
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_kernel(const float* __restrict__ qkv, const int* __restrict__ slots, const int* __restrict__ positions,
                 T* __restrict__ cache_k, T* __restrict__ cache_v, int layer, int n_slots, int S, int d, int rows) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int s = slots[r], pos = positions[r];
  if (s < 0 || s >= n_slots || pos < 0 || pos >= S) return;
  const int64_t base = (((int64_t)layer * n_slots + s) * S + pos) * d;
  const float* src = qkv + (int64_t)r * 3 * d;
  for (int i = threadIdx.x; i < d; i += 256) {
    cache_k[base + i] = from_f<T>(src[d + i]);
    cache_v[base + i] = from_f<T>(src[2 * d + i]);
  }
}

// conv1 operand: col[(b, t), tap * n_mels + c] = mel[b, c, t + tap - 1] (zero outside).
// A 32-frame tile of all channels goes through shared memory so that both the
// read (time-major) and the write (channel-major) are coalesced.
template <typename T>
__global__ void __launch_bounds__(256)
im2col_conv1_kernel(const float* __restrict__ mel, T* __restrict__ col, int n_mels, int frames) {
  extern __shared__ float tile[];  // [n_mels][35]
  const int b = blockIdx.y, t0 = blockIdx.x * 32;
  for (int i = threadIdx.x; i < n_mels * 34; i += 256) {
    const int c = i / 34, j = i % 34, t = t0 + j - 1;
    tile[c * 35 + j] = (t >= 0 && t < frames) ? mel[((int64_t)b * n_mels + c) * frames + t] : 0.0f;
  }
  __syncthreads();
  const int K = 3 * n_mels;
  for (int i = threadIdx.x; i < 32 * K; i += 256) {
    const int tl = i / K, kk = i % K, tap = kk / n_mels, c = kk % n_mels;
    if (t0 + tl < frames)
      col[((int64_t)b * frames + t0 + tl) * K + kk] = from_f<T>(tile[c * 35 + tl + tap]);
  }
}

template <typename T>
__global__ void zero_rows_kernel(T* __restrict__ p, int64_t bstride, int64_t row_off, int d, int B) {
  const int b = blockIdx.x;
  if (b >= B) return;
  for (int i = threadIdx.x; i < d; i += blockDim.x) p[b * bstride + row_off + i] = from_f<T>(0.0f);
}

}  // namespace wdz
