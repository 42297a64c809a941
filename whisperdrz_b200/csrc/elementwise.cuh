// Row-wise helpers around the GEMMs: LayerNorm over the fp32 residual stream
// (src/whisperdrz/model.py:195-200, eps 1e-5), token + learned positional
// embedding (model.py:597), the conv1 im2col (model.py:449,467), K/V append
// into the slotted self-attention cache (model.py:51-54) and slot bookkeeping.
#pragma once
#include "common.cuh"

namespace wdz {

// Four consecutive parameters / outputs at once (16 bytes of fp32 or 8 bytes of bf16).
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 t = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
  const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// y[r] = LN(x[src(r)]) * gamma + beta over the fp32 residual stream, d % 4 == 0, d <= 2048.
// Two shapes of the same arithmetic (mean, then centred variance, both from registers; the row is
// read once): one warp per row for the tens of thousands of encoder rows, and one 128-thread CTA per
// row for the few decode rows, where the time is a chain of memory latencies, not bandwidth - there
// every thread issues its (at most four) loads of x, gamma and beta at once.
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
      float g[4], bt[4], o[4];
      load4(gamma + 4 * j, g);
      load4(beta + 4 * j, bt);
      o[0] = (v[i].x - mean) * rstd * g[0] + bt[0];
      o[1] = (v[i].y - mean) * rstd * g[1] + bt[1];
      o[2] = (v[i].z - mean) * rstd * g[2] + bt[2];
      o[3] = (v[i].w - mean) * rstd * g[3] + bt[3];
      store4(yr + 4 * j, o);
    }
  }
}

template <typename TP, typename TO>
__global__ void __launch_bounds__(128)
layernorm_row_kernel(const float* __restrict__ x, int64_t ldx, const int* __restrict__ row_idx,
                     const TP* __restrict__ gamma, const TP* __restrict__ beta,
                     TO* __restrict__ y, int64_t ldy, int rows, int d,
                     float* __restrict__ zero = nullptr, int64_t ldz = 0, int nz = 0) {
  pdl_trigger();
  constexpr int MAXI = 4;  // float4 per thread: d <= 2048
  __shared__ float red[2][4];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nv = d >> 2;
  // gamma and beta do not depend on the previous kernel: fetch them before waiting for it
  float g[MAXI][4], bt[MAXI][4];
#pragma unroll
  for (int i = 0; i < MAXI; ++i) {
    const int j = tid + 128 * i;
    if (j < nv) { load4(gamma + 4 * j, g[i]); load4(beta + 4 * j, bt[i]); }
  }
  pdl_wait();
  // optional: clear row r of an fp32 buffer that the next product accumulates into (K-split partial sums)
  if (zero)
    for (int j = tid; j < (nz >> 2); j += 128) reinterpret_cast<float4*>(zero + (int64_t)r * ldz)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)(row_idx ? row_idx[r] : r) * ldx);
  float4 v[MAXI];
#pragma unroll
  for (int i = 0; i < MAXI; ++i) {
    const int j = tid + 128 * i;
    v[i] = j < nv ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXI; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  s = warp_sum(s);
  if (lane == 0) red[0][warp] = s;
  __syncthreads();
  const float mean = ((red[0][0] + red[0][1]) + (red[0][2] + red[0][3])) / d;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXI; ++i) {
    if (tid + 128 * i < nv) {
      const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      q += a * a + b * b + c * c + e * e;
    }
  }
  q = warp_sum(q);
  if (lane == 0) red[1][warp] = q;
  __syncthreads();
  const float rstd = rsqrtf(((red[1][0] + red[1][1]) + (red[1][2] + red[1][3])) / d + 1e-5f);
  TO* yr = y + (int64_t)r * ldy;
#pragma unroll
  for (int i = 0; i < MAXI; ++i) {
    const int j = tid + 128 * i;
    if (j < nv) {
      float o[4];
      o[0] = (v[i].x - mean) * rstd * g[i][0] + bt[i][0];
      o[1] = (v[i].y - mean) * rstd * g[i][1] + bt[i][1];
      o[2] = (v[i].z - mean) * rstd * g[i][2] + bt[i][2];
      o[3] = (v[i].w - mean) * rstd * g[i][3] + bt[i][3];
      store4(yr + 4 * j, o);
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

// f32 [n, ld_src] (first d columns) -> bf16 [n, ld_dst]; one block per row.
__global__ void cast_rows_kernel(const float* __restrict__ src, int64_t ld_src, bf16* __restrict__ dst, int64_t ld_dst,
                                 int n, int d) {
  const int r = blockIdx.x;
  if (r >= n) return;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)r * ld_src + c);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst + (int64_t)r * ld_dst + c) = o;
  }
}

}  // namespace wdz
