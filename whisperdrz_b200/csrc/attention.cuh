// Attention kernels (head_dim 64, scale 1/8, fp32 softmax and accumulation).
//
//   attn_enc_simt_kernel - encoder self-attention, non-causal, flash-style
//       tiling on the CUDA cores (MultiHeadAttention.qkv_attention,
//       src/whisperdrz/model.py:276-298).  fp32-mode arithmetic and bf16 fallback.
//   attn_dec_kernel / attn_dec_combine_kernel - one query row against a slot of
//       the KV cache, split over the key axis; serves both the ragged causal
//       self-attention (keys [0, position]) and the cross-attention over all
//       encoder positions (model.py:20-76, 336-359).  HBM-bound: every K and V
//       element of the attended range is read exactly once per row, with
//       16-byte loads that cover whole 128-byte head vectors.
#pragma once
#include "common.cuh"

namespace wdz {

constexpr int HD = 64;
constexpr float QK_SCALE_LOG2E = 0.125f * 1.4426950408889634f;

template <typename T>
__global__ void __launch_bounds__(256)
attn_enc_simt_kernel(const T* __restrict__ qkv, T* __restrict__ out, int Tn, int d) {
  extern __shared__ float sm[];
  constexpr int LD = 65;
  float* Qs = sm;
  float* Ks = Qs + 64 * LD;
  float* Vs = Ks + 64 * LD;
  float* Ps = Vs + 64 * LD;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int q0 = blockIdx.x * 64, h = blockIdx.y, b = blockIdx.z;
  const int64_t row0 = (int64_t)b * Tn;
  const int ld = 3 * d;

  for (int i = tid; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    Qs[r * LD + c] = q0 + r < Tn ? to_f(qkv[(row0 + q0 + r) * ld + h * HD + c]) * QK_SCALE_LOG2E : 0.0f;
  }
  float m_run[4], l_run[4], o[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
  }

  for (int k0 = 0; k0 < Tn; k0 += 64) {
    __syncthreads();  // previous tile fully consumed (and Q visible on the first pass)
    for (int i = tid; i < 64 * 64; i += 256) {
      const int r = i >> 6, c = i & 63;
      const bool ok = k0 + r < Tn;
      const int64_t base = (row0 + k0 + r) * ld + h * HD + c;
      Ks[r * LD + c] = ok ? to_f(qkv[base + d]) : 0.0f;
      Vs[r * LD + c] = ok ? to_f(qkv[base + 2 * d]) : 0.0f;
    }
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll 8
    for (int c = 0; c < HD; ++c) {
      float a[4], k[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Qs[(ty + 16 * i) * LD + c];
#pragma unroll
      for (int j = 0; j < 4; ++j) k[j] = Ks[(tx + 16 * j) * LD + c];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(a[i], k[j], s[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (k0 + tx + 16 * j >= Tn) s[i][j] = -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
      const float m_new = fmaxf(m_run[i], mx);
      const float alpha = exp2f(m_run[i] - m_new);  // first tile: exp2(-inf) = 0
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = exp2f(s[i][j] - m_new);
        Ps[(ty + 16 * i) * LD + tx + 16 * j] = p;
        sum += p;
      }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
      l_run[i] = l_run[i] * alpha + sum;
      m_run[i] = m_new;
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] *= alpha;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 64; ++k) {
      float p[4], v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = Ps[(ty + 16 * i) * LD + k];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = Vs[k * LD + tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = fmaf(p[i], v[j], o[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = q0 + ty + 16 * i;
    if (r >= Tn) continue;
    const float inv = 1.0f / l_run[i];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      out[(row0 + r) * d + h * HD + tx + 16 * j] = from_f<T>(o[i][j] * inv);
  }
}

inline size_t attn_enc_simt_smem() { return sizeof(float) * 4 * 64 * 65; }

struct AttnDecParams {
  const float* q; int64_t ldq;      // query of row r, head h at q + r * ldq + h * 64
  const void* cache_k; const void* cache_v;
  int layer, n_slots, S, d;         // cache [layers, n_slots, S, d]
  const int* slots; const int* positions; int fixed_len;  // len = positions ? positions[r] + 1 : fixed_len
  int chunk, max_splits;
  float* part_o; float* part_ml;    // [rows, max_splits, H, 64] and [rows, max_splits, H, 2]
  float* out; int64_t ldo;          // combine: out + r * ldo + h * 64
};

// Block = H warps (warp = head); grid = (splits, rows).
template <typename T>
__global__ void attn_dec_kernel(AttnDecParams p) {
  constexpr int VEC = Vec<T>::N;   // elements per 16-byte piece
  constexpr int LPK = HD / VEC;    // lanes covering one key's head vector
  constexpr int KPI = 32 / LPK;    // keys per warp iteration
  const int r = blockIdx.y, split = blockIdx.x;
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31, H = blockDim.x >> 5;
  const int slot = p.slots[r];
  if (slot < 0 || slot >= p.n_slots) return;
  int len = p.positions ? p.positions[r] + 1 : p.fixed_len;
  len = len > p.S ? p.S : len;
  const int start = split * p.chunk;
  if (start >= len) return;
  const int end = min(len, start + p.chunk);
  const int piece = lane % LPK, grp = lane / LPK;

  float qv[VEC];
  {
    const float* qp = p.q + (int64_t)r * p.ldq + h * HD + piece * VEC;
#pragma unroll
    for (int e = 0; e < VEC; ++e) qv[e] = qp[e] * QK_SCALE_LOG2E;
  }
  const int64_t base = (((int64_t)p.layer * p.n_slots + slot) * p.S) * p.d + h * HD + piece * VEC;
  const T* K = reinterpret_cast<const T*>(p.cache_k) + base;
  const T* V = reinterpret_cast<const T*>(p.cache_v) + base;

  float m = -INFINITY, l = 0.0f, o[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) o[e] = 0.0f;

  for (int t0 = start; t0 < end; t0 += 2 * KPI) {
    const int ta = t0 + grp, tb = t0 + KPI + grp;
    const bool va = ta < end, vb = tb < end;
    float ka[VEC], kb[VEC], xa[VEC], xb[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) ka[e] = kb[e] = xa[e] = xb[e] = 0.0f;
    if (va) { load_vec_nc(K + (int64_t)ta * p.d, ka); load_vec_nc(V + (int64_t)ta * p.d, xa); }
    if (vb) { load_vec_nc(K + (int64_t)tb * p.d, kb); load_vec_nc(V + (int64_t)tb * p.d, xb); }
    float sa = 0.0f, sb = 0.0f;
#pragma unroll
    for (int e = 0; e < VEC; ++e) { sa = fmaf(qv[e], ka[e], sa); sb = fmaf(qv[e], kb[e], sb); }
#pragma unroll
    for (int o2 = LPK / 2; o2 > 0; o2 >>= 1) {
      sa += __shfl_xor_sync(0xffffffffu, sa, o2);
      sb += __shfl_xor_sync(0xffffffffu, sb, o2);
    }
    if (!va) sa = -INFINITY;
    if (!vb) sb = -INFINITY;
    const float m_new = fmaxf(m, fmaxf(sa, sb));
    if (m_new > -INFINITY) {
      const float alpha = exp2f(m - m_new);
      const float pa = exp2f(sa - m_new), pb = exp2f(sb - m_new);
      l = l * alpha + pa + pb;
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = fmaf(pb, xb[e], fmaf(pa, xa[e], o[e] * alpha));
      m = m_new;
    }
  }
  // merge the key sub-groups of the warp
#pragma unroll
  for (int o2 = LPK; o2 < 32; o2 <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o2);
    const float l2 = __shfl_xor_sync(0xffffffffu, l, o2);
    const float m_new = fmaxf(m, m2);
    const float a1 = m_new > -INFINITY ? exp2f(m - m_new) : 0.0f;
    const float a2 = m_new > -INFINITY ? exp2f(m2 - m_new) : 0.0f;
    l = l * a1 + l2 * a2;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float o2v = __shfl_xor_sync(0xffffffffu, o[e], o2);
      o[e] = o[e] * a1 + o2v * a2;
    }
    m = m_new;
  }
  const int64_t pi = ((int64_t)r * p.max_splits + split) * H + h;
  if (grp == 0) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) p.part_o[pi * HD + piece * VEC + e] = o[e];
  }
  if (lane == 0) { p.part_ml[pi * 2] = m; p.part_ml[pi * 2 + 1] = l; }
}

// Block = H warps; grid = rows.  Merges the splits that the row's length makes valid.
__global__ void attn_dec_combine_kernel(AttnDecParams p) {
  const int r = blockIdx.x;
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31, H = blockDim.x >> 5;
  const int slot = p.slots[r];
  if (slot < 0 || slot >= p.n_slots) return;
  int len = p.positions ? p.positions[r] + 1 : p.fixed_len;
  len = len > p.S ? p.S : len;
  const int nsplit = (len + p.chunk - 1) / p.chunk;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s)
    M = fmaxf(M, p.part_ml[(((int64_t)r * p.max_splits + s) * H + h) * 2]);
  float L = 0.0f, o0 = 0.0f, o1 = 0.0f;
  for (int s = 0; s < nsplit; ++s) {
    const int64_t pi = ((int64_t)r * p.max_splits + s) * H + h;
    const float w = exp2f(p.part_ml[pi * 2] - M);
    L = fmaf(p.part_ml[pi * 2 + 1], w, L);
    o0 = fmaf(p.part_o[pi * HD + lane], w, o0);
    o1 = fmaf(p.part_o[pi * HD + 32 + lane], w, o1);
  }
  const float inv = L > 0.0f ? 1.0f / L : 0.0f;
  float* dst = p.out + (int64_t)r * p.ldo + h * HD;
  dst[lane] = o0 * inv;
  dst[32 + lane] = o1 * inv;
}

}  // namespace wdz
