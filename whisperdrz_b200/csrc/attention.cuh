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
#include "../../include/wdz.h"
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
  int rows;                         // rows of the launch (the kernel walks max_splits x rows items)
  int split_major;                  // item order: 1 = all rows of range 0, then range 1, ... (persistent walk: the ranges
                                    // every row has come first); 0 = the ranges of a row side by side (one CTA per item)
  float* part_o; float* part_ml;    // [rows, max_splits, H, 64] and [rows, max_splits, H, 2]
  void* out; int64_t ldo;           // combine: out (TO) + r * ldo + h * 64
  int* counters;                    // [rows], zero between launches: split CTAs of a row count themselves in, the
                                    // last one merges the row's partial results (nullptr: a combine launch follows)
};

// Block = a group of heads (warp = head); grid = (splits, rows, head groups).
// The K/V loads of the next 2*KPI keys are issued before the current ones are
// consumed, so every lane keeps eight 16-byte loads in flight.
template <typename T>
__global__ void __launch_bounds__(256) attn_dec_kernel(AttnDecParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int VEC = Vec<T>::N;   // elements per 16-byte piece
  constexpr int LPK = HD / VEC;    // lanes covering one key's head vector
  constexpr int KPI = 32 / LPK;    // keys per warp load
  constexpr int STEP = 2 * KPI;    // keys per loop iteration
  const int r = blockIdx.y, split = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int h = blockIdx.z * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int H = gridDim.z * (blockDim.x >> 5);
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

  float ka[VEC], kb[VEC], xa[VEC], xb[VEC];      // current keys / values
  float nka[VEC], nkb[VEC], nxa[VEC], nxb[VEC];  // next iteration's
  auto fetch = [&](int t0, float (&k0)[VEC], float (&k1)[VEC], float (&v0)[VEC], float (&v1)[VEC]) {
    const int ta = t0 + grp, tb = t0 + KPI + grp;
#pragma unroll
    for (int e = 0; e < VEC; ++e) k0[e] = k1[e] = v0[e] = v1[e] = 0.0f;
    if (ta < end) { load_vec_nc(K + (int64_t)ta * p.d, k0); load_vec_nc(V + (int64_t)ta * p.d, v0); }
    if (tb < end) { load_vec_nc(K + (int64_t)tb * p.d, k1); load_vec_nc(V + (int64_t)tb * p.d, v1); }
  };
  fetch(start, ka, kb, xa, xb);
  for (int t0 = start; t0 < end; t0 += STEP) {
    if (t0 + STEP < end) fetch(t0 + STEP, nka, nkb, nxa, nxb);
    const bool va = t0 + grp < end, vb = t0 + KPI + grp < end;
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
#pragma unroll
    for (int e = 0; e < VEC; ++e) { ka[e] = nka[e]; kb[e] = nkb[e]; xa[e] = nxa[e]; xb[e] = nxb[e]; }
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

// Streaming variant for long, fixed-length ranges (cross-attention): the K and
// V rows of a CTA's key range are contiguous in the cache ([keys, d]), so a
// producer warp moves them into a ring of shared-memory stages with bulk
// asynchronous copies (cp.async.bulk + mbarrier transaction counts) and the H
// head warps consume them from shared memory.  Bytes in flight per SM are set
// by the ring (STAGES x 2 x SK x d elements), not by registers.
// Block = (H + 1) warps; grid = (splits, rows).  Waits are bounded.
constexpr int ATT_STAGES = 4;
constexpr long long ATT_WAIT_CYCLES = 2000000000ll;

__device__ __forceinline__ uint32_t att_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool att_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, DevStatus* status) {
  const uint32_t a = att_smem_u32(bar);
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
      if (clock64() - t0 > ATT_WAIT_CYCLES) {
        *abort_flag = 1;
        if (status) { atomicCAS(&status->code, 0, WDZ_ETIMEOUT); status->detail = 1000000 + (int)blockIdx.x; }
        return false;
      }
    }
  }
}

template <typename TO>
__device__ __forceinline__ void attn_dec_merge_head(const AttnDecParams& p, int r, int h, int lane, int H, int nsplit);

template <typename T>
__global__ void __launch_bounds__(672, 1) attn_dec_stream_kernel(AttnDecParams p, DevStatus* status) {
  constexpr int VEC = Vec<T>::N;
  constexpr int LPK = HD / VEC;
  constexpr int KPI = 32 / LPK;
  constexpr int SK = 2 * KPI;      // keys per stage: one consumer iteration
  extern __shared__ __align__(128) uint8_t att_smem[];
  __shared__ int s_last;
  const int H = (blockDim.x >> 5) - 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t half_bytes = (size_t)SK * p.d * sizeof(T);          // K (or V) bytes of one stage
  uint64_t* bars = reinterpret_cast<uint64_t*>(att_smem + ATT_STAGES * 2 * half_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + ATT_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * ATT_STAGES);

  pdl_trigger();
  const int n_items = p.max_splits * p.rows;
  const bool one_item = (int)gridDim.x >= n_items;   // one CTA per item: most self-attention items lie past their
  if (one_item) {                                    // row's length, and those CTAs should leave before any set-up
    pdl_wait();
    const int item = blockIdx.x;
    const int split = p.split_major ? item / p.rows : item % p.max_splits;
    const int r = p.split_major ? item - split * p.rows : item / p.max_splits;
    const int slot = p.slots[r];
    int len = p.positions ? p.positions[r] + 1 : p.fixed_len;
    len = len > p.S ? p.S : len;
    if (slot < 0 || slot >= p.n_slots || split * p.chunk >= len) return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < ATT_STAGES; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(att_smem_u32(full + i)), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(att_smem_u32(empty + i)), "r"(H));
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (!one_item) pdl_wait();     // the persistent walk sets its ring up while the previous kernel drains

  // The CTA walks the work items (key range `split` of row r) that fall to it - all of them when the grid is one
  // CTA per SM, exactly one when the grid is one CTA per item - and the ring keeps running across items: the producer is already
  // fetching the next item's keys while the head warps finish the current one.  `it` counts ring stages over the
  // whole walk; producer and consumers step through the same items, so they agree on it.
  int it = 0;
  if (warp == H) {
    if (lane == 0) {
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int split = p.split_major ? item / p.rows : item % p.max_splits;
        const int r = p.split_major ? item - split * p.rows : item / p.max_splits;
        const int slot = p.slots[r];
        int len = p.positions ? p.positions[r] + 1 : p.fixed_len;
        len = len > p.S ? p.S : len;
        const int start = split * p.chunk;
        if (slot < 0 || slot >= p.n_slots || start >= len) continue;
        const int end = min(len, start + p.chunk);
        const int n_iter = (end - start + SK - 1) / SK;
        const int64_t row_base = (((int64_t)p.layer * p.n_slots + slot) * p.S) * p.d;
        const T* Kg = reinterpret_cast<const T*>(p.cache_k) + row_base;
        const T* Vg = reinterpret_cast<const T*>(p.cache_v) + row_base;
        bool ok = true;
        for (int j = 0; j < n_iter; ++j, ++it) {
          const int stage = it % ATT_STAGES;
          const uint32_t phase = (it / ATT_STAGES) & 1;
          if (!(ok = att_mbar_wait(empty + stage, phase ^ 1, abort_flag, status))) break;
          const int t = start + j * SK;
          const uint32_t bytes = (uint32_t)((size_t)min(SK, end - t) * p.d * sizeof(T));
          uint8_t* dstk = att_smem + (size_t)stage * 2 * half_bytes;
          const uint32_t bar = att_smem_u32(full + stage);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(att_smem_u32(dstk)), "l"(Kg + (int64_t)t * p.d), "r"(bytes), "r"(bar) : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(att_smem_u32(dstk + half_bytes)), "l"(Vg + (int64_t)t * p.d), "r"(bytes), "r"(bar) : "memory");
        }
        if (!ok) break;
      }
    }
    return;
  }

  const int h = warp;
  const int piece = lane % LPK, grp = lane / LPK;
  const int col = h * HD + piece * VEC;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int split = p.split_major ? item / p.rows : item % p.max_splits;
        const int r = p.split_major ? item - split * p.rows : item / p.max_splits;
    const int slot = p.slots[r];
    int len = p.positions ? p.positions[r] + 1 : p.fixed_len;
    len = len > p.S ? p.S : len;
    const int start = split * p.chunk;
    if (slot < 0 || slot >= p.n_slots || start >= len) continue;   // uniform over the CTA
    const int end = min(len, start + p.chunk);
    const int n_iter = (end - start + SK - 1) / SK;
    float qv[VEC];
    {
      const float* qp = p.q + (int64_t)r * p.ldq + h * HD + piece * VEC;
#pragma unroll
      for (int e = 0; e < VEC; ++e) qv[e] = qp[e] * QK_SCALE_LOG2E;
    }
    float m = -INFINITY, l = 0.0f, o[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) o[e] = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_iter; ++j, ++it) {
      const int stage = it % ATT_STAGES;
      const uint32_t phase = (it / ATT_STAGES) & 1;
      ok = att_mbar_wait(full + stage, phase, abort_flag, status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const T* Ks = reinterpret_cast<const T*>(att_smem + (size_t)stage * 2 * half_bytes);
      const T* Vs = reinterpret_cast<const T*>(att_smem + (size_t)stage * 2 * half_bytes + half_bytes);
      const int t0 = start + j * SK;
      const bool va = t0 + grp < end, vb = t0 + KPI + grp < end;
      float ka[VEC], kb[VEC], xa[VEC], xb[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) ka[e] = kb[e] = xa[e] = xb[e] = 0.0f;
      if (va) { load_vec(Ks + (size_t)grp * p.d + col, ka); load_vec(Vs + (size_t)grp * p.d + col, xa); }
      if (vb) { load_vec(Ks + (size_t)(KPI + grp) * p.d + col, kb); load_vec(Vs + (size_t)(KPI + grp) * p.d + col, xb); }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(att_smem_u32(empty + stage)) : "memory");
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
    // (after an exhausted wait the warps still meet at the barrier below and leave together from there)
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
    // The items of a row count themselves in; whichever comes last finds all partial results in place and merges
    // them, so no combine launch is needed and nobody waits for anybody.
    const int nsplit = (len + p.chunk - 1) / p.chunk;
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"r"(H * 32) : "memory");          // the H head warps; the producer warp is not part of it
    if (threadIdx.x == 0) {
      if (*abort_flag) {
        s_last = -1;      // a wait ran out somewhere in this CTA: the status word tells the host that the output is
                          // void (it clears the arrival counters when it reads that status); everybody leaves
      } else {
        const int old = atomicAdd(p.counters + r, 1);
        s_last = old == nsplit - 1;
        if (s_last) p.counters[r] = 0;                                 // ready for the next launch
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(H * 32) : "memory");
    const int last = s_last;
    if (last < 0) return;
    if (last) {
      __threadfence();
      attn_dec_merge_head<T>(p, r, h, lane, H, nsplit);
    }
  }
}

template <typename T>
inline size_t attn_dec_stream_smem(int d) {
  return (size_t)ATT_STAGES * 2 * (2 * (32 / (HD / Vec<T>::N))) * d * sizeof(T) + 2 * ATT_STAGES * 8 + 16;
}

// Merges the nsplit partial results of (row r, head h) and writes the normalised output; one warp per head.
// Partials written by other CTAs are read past L1 (ld.global.cg).
template <typename TO>
__device__ __forceinline__ void attn_dec_merge_head(const AttnDecParams& p, int r, int h, int lane, int H, int nsplit) {
  const int64_t base = (int64_t)r * p.max_splits * H + h;   // entry of split s: base + s * H
  float o0 = 0.0f, o1 = 0.0f, L = 0.0f, M = -INFINITY;
  // splits in groups of 32: lanes fetch (m, l) of different splits in parallel
  for (int s0 = 0; s0 < nsplit; s0 += 32) {
    const int s = s0 + lane;
    float ms = -INFINITY, ls = 0.0f;
    if (s < nsplit) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (base + (int64_t)s * H) * 2));
      ms = ml.x; ls = ml.y;
    }
    const float M_new = fmaxf(M, warp_max(ms));
    const float resc = exp2f(M - M_new);          // 0 on the first group
    const float w = s < nsplit ? exp2f(ms - M_new) : 0.0f;
    L = L * resc + warp_sum(ls * w);
    o0 *= resc; o1 *= resc;
    const int cnt = min(32, nsplit - s0);
    // sixteen splits at a time: all their loads are issued before the first one is used
    for (int i0 = 0; i0 < cnt; i0 += 16) {
      float x0[16], x1[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const bool ok = i0 + u < cnt;
        const float* po = p.part_o + (base + (int64_t)(s0 + (ok ? i0 + u : 0)) * H) * HD;
        x0[u] = ok ? __ldcg(po + lane) : 0.0f;
        x1[u] = ok ? __ldcg(po + 32 + lane) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const float wi = __shfl_sync(0xffffffffu, w, (i0 + u) & 31);
        o0 = fmaf(x0[u], wi, o0);
        o1 = fmaf(x1[u], wi, o1);
      }
    }
    M = M_new;
  }
  const float inv = L > 0.0f ? 1.0f / L : 0.0f;
  TO* dst = reinterpret_cast<TO*>(p.out) + (int64_t)r * p.ldo + h * HD;
  dst[lane] = from_f<TO>(o0 * inv);
  dst[32 + lane] = from_f<TO>(o1 * inv);
}

// Block = H warps; grid = rows.  Merges the splits that the row's length makes valid.
template <typename TO>
__global__ void attn_dec_combine_kernel(AttnDecParams p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31, H = blockDim.x >> 5;
  const int slot = p.slots[r];
  if (slot < 0 || slot >= p.n_slots) return;
  int len = p.positions ? p.positions[r] + 1 : p.fixed_len;
  len = len > p.S ? p.S : len;
  attn_dec_merge_head<TO>(p, r, h, lane, H, (len + p.chunk - 1) / p.chunk);
}

}  // namespace wdz
