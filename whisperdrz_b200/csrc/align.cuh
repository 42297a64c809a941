// Word-timing alignment: the device steps of fill_word_timings_batch
// (src/whisperdrz/dtw_align.py:1112-1240).
//
//   align_rows_kernel      rows of a teacher-forced pass: chunk b, token t -> (slot, position)
//   align_capture_kernel   keeps the cross-attention queries of the alignment heads
//                          (CrossAttnCapture, dtw_align.py:498-551)
//   align_scores_kernel    QK^T of one (chunk, head) against the slot's cached cross keys,
//                          softmax over the audio columns below the chunk's cap
//                          (compute_attention :553-586, _dtw_prep_batch :725-727)
//   align_colstats_kernel  mean and 1/std over the chunk's valid text rows per (head, column) (:729-737)
//   align_matrix_kernel    normalise, 7-wide median along audio with reflect padding, mean over
//                          heads (:739-744; replaces the reference's Triton median kernel)
//   dtw_kernel             cost accumulation by anti-diagonals with the trace kept in shared
//                          memory (2 bits per cell) and the backtrace (_dtw_numba :170-223),
//                          anchor bands as an allowed column range per row (_apply_anchor_bands :589-641)
#pragma once
#include "common.cuh"
#include "../../include/wdz.h"

namespace wdz {

constexpr int ALIGN_MAX_HEADS = 16;
constexpr int ALIGN_HD = 64;

struct AlignHeads {
  int n;
  int layer[ALIGN_MAX_HEADS];
  int head[ALIGN_MAX_HEADS];
};

// Row r of the pass is token t = (r0 + r) % t_pad of chunk b = (r0 + r) / t_pad; rows past the chunk's
// length get slot -1, which every kernel of the pass skips.
__global__ void align_rows_kernel(const int* __restrict__ chunk_slots, const int* __restrict__ chunk_lens, int t_pad,
                                  int r0, int n, int n_slots, int* __restrict__ slots, int* __restrict__ positions) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int b = (r0 + r) / t_pad, t = (r0 + r) % t_pad;
  const int s = chunk_slots[b];
  slots[r] = (t < chunk_lens[b] && s >= 0 && s < n_slots) ? s : -1;
  positions[r] = t;
}

// q [n, ldq] of layer `layer` -> qcap[j][row_base + r][64] (f32) for every selected head j of that layer.
template <typename TQ>
__global__ void align_capture_kernel(const TQ* __restrict__ q, int64_t ldq, int n, int layer, AlignHeads hs,
                                     float* __restrict__ qcap, int64_t rows_total, int64_t row_base) {
  const int r = blockIdx.x;
  const int e = threadIdx.x & 63, which = threadIdx.x >> 6;   // blockDim = 64 * heads of this layer (<= 1024)
  int seen = 0;
  for (int j = 0; j < hs.n; ++j) {
    if (hs.layer[j] != layer) continue;
    if (seen++ == which) {
      qcap[((int64_t)j * rows_total + row_base + r) * ALIGN_HD + e] = to_f(q[(int64_t)r * ldq + hs.head[j] * ALIGN_HD + e]);
      return;
    }
  }
}

// q sits in shared memory (one row per warp) and is read 16 bytes at a time.
__device__ __forceinline__ float dot64(const float* __restrict__ q, const float* __restrict__ k) {
  float s = 0.0f;
#pragma unroll
  for (int e = 0; e < ALIGN_HD; e += 4) {
    const float4 kv = *reinterpret_cast<const float4*>(k + e);
    const float4 qv = *reinterpret_cast<const float4*>(q + e);
    s += qv.x * kv.x + qv.y * kv.y + qv.z * kv.z + qv.w * kv.w;
  }
  return s;
}
__device__ __forceinline__ float dot64(const float* __restrict__ q, const bf16* __restrict__ k) {
  float s = 0.0f;
#pragma unroll
  for (int e = 0; e < ALIGN_HD; e += 8) {
    float kv[8];
    load_vec(k + e, kv);
    const float4 qa = *reinterpret_cast<const float4*>(q + e), qb = *reinterpret_cast<const float4*>(q + e + 4);
    s += qa.x * kv[0] + qa.y * kv[1] + qa.z * kv[2] + qa.w * kv[3] + qb.x * kv[4] + qb.y * kv[5] + qb.z * kv[6] + qb.w * kv[7];
  }
  return s;
}

// One warp per text row: lane a handles columns a, a + 32, ...; the row's scores stay in registers
// (ceil(Ta / 32) <= ALIGN_COLS_PER_LANE), softmax over columns < cap, zeros from cap on.
// grid = (ceil(t_pad / 8), heads, chunks), block = 256.  The lens / slots / caps pointers and w start at the
// first chunk of this launch; qcap is indexed with the chunk's number in the whole pass (chunk0 + b).
constexpr int ALIGN_COLS_PER_LANE = 48;   // Ta <= 1536
template <typename T>
__global__ void __launch_bounds__(256)
align_scores_kernel(const float* __restrict__ qcap, int64_t rows_total, int chunk0, int t_pad, const int* __restrict__ chunk_lens,
                    const int* __restrict__ chunk_slots, const int* __restrict__ caps, AlignHeads hs,
                    const T* __restrict__ cross_k, int n_slots, int Ta, int d, float* __restrict__ w) {
  __shared__ __align__(16) float qs[8][ALIGN_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp, j = blockIdx.y, b = blockIdx.z;
  const int slot = chunk_slots[b];
  const bool live = t < chunk_lens[b] && t < t_pad && slot >= 0 && slot < n_slots;   // uniform over the warp
  if (live && lane < 16)
    *reinterpret_cast<float4*>(&qs[warp][lane * 4]) =
        *reinterpret_cast<const float4*>(qcap + ((int64_t)j * rows_total + (int64_t)(chunk0 + b) * t_pad + t) * ALIGN_HD + lane * 4);
  __syncwarp();
  if (!live) return;
  const int cap = min(max(caps[b], 0), Ta);
  const T* kbase = cross_k + (((int64_t)hs.layer[j] * n_slots + slot) * Ta) * d + hs.head[j] * ALIGN_HD;
  const float scale = 0.125f;                       // hd^-0.25 on each side (dtw_align.py:563)
  float s[ALIGN_COLS_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int c = 0; c < ALIGN_COLS_PER_LANE; ++c) {
    const int a = c * 32 + lane;
    s[c] = -INFINITY;
    if (a < cap) {
      s[c] = dot64(qs[warp], kbase + (int64_t)a * d) * scale;
      mx = fmaxf(mx, s[c]);
    }
  }
  mx = warp_max(mx);
  float sum = 0.0f;
#pragma unroll
  for (int c = 0; c < ALIGN_COLS_PER_LANE; ++c) {
    const int a = c * 32 + lane;
    s[c] = a < cap ? expf(s[c] - mx) : 0.0f;
    sum += s[c];
  }
  sum = warp_sum(sum);
  const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
  float* wr = w + (((int64_t)b * hs.n + j) * t_pad + t) * Ta;
#pragma unroll
  for (int c = 0; c < ALIGN_COLS_PER_LANE; ++c) {
    const int a = c * 32 + lane;
    if (a < Ta) wr[a] = s[c] * inv;
  }
}

// mean[b][j][a] and rstd[b][j][a] over text rows t < len_b (population variance, floor 1e-12).
// grid = (ceil(Ta / 128), heads, chunks), block = 128.
__global__ void align_colstats_kernel(const float* __restrict__ w, int n_heads, int t_pad, int Ta,
                                      const int* __restrict__ chunk_lens, float* __restrict__ mean,
                                      float* __restrict__ rstd) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x, j = blockIdx.y, b = blockIdx.z;
  if (a >= Ta) return;
  const int len = min(chunk_lens[b], t_pad);
  const float* col = w + (((int64_t)b * n_heads + j) * t_pad) * Ta + a;
  float sum = 0.0f;
  for (int t = 0; t < len; ++t) sum += col[(int64_t)t * Ta];
  const float n = (float)max(len, 1);
  const float m = sum / n;
  float var = 0.0f;
  for (int t = 0; t < len; ++t) {
    const float dlt = col[(int64_t)t * Ta] - m;
    var += dlt * dlt;
  }
  var = fmaxf(var / n, 1e-12f);
  const int64_t o = ((int64_t)b * n_heads + j) * Ta + a;
  mean[o] = m;
  rstd[o] = 1.0f / sqrtf(var);
}

__device__ __forceinline__ void cswap(float& x, float& y) {
  const float lo = fminf(x, y), hi = fmaxf(x, y);
  x = lo; y = hi;
}
// Median of seven by a selection network (only the middle element is completed).
__device__ __forceinline__ float median7(float v0, float v1, float v2, float v3, float v4, float v5, float v6) {
  cswap(v0, v5); cswap(v0, v3); cswap(v1, v6); cswap(v2, v4); cswap(v0, v1); cswap(v3, v5);
  cswap(v2, v6); cswap(v2, v3); cswap(v3, v6); cswap(v4, v5); cswap(v1, v4); cswap(v1, v3); cswap(v3, v4);
  return v3;
}

// out[b][t][a] = mean over heads of median7 over a' of (w[b][j][t][a'] - mean[b][j][a']) * rstd[b][j][a'],
// a' = a-3..a+3 reflected at 0 and Ta-1.  Rows t >= len_b are zero.  grid = (t_pad, chunks), block = 256.
__global__ void __launch_bounds__(256)
align_matrix_kernel(const float* __restrict__ w, const float* __restrict__ mean, const float* __restrict__ rstd,
                    int n_heads, int t_pad, int Ta, const int* __restrict__ chunk_lens, float* __restrict__ out) {
  const int t = blockIdx.x, b = blockIdx.y;
  float* orow = out + ((int64_t)b * t_pad + t) * Ta;
  if (t >= chunk_lens[b]) {
    for (int a = threadIdx.x; a < Ta; a += blockDim.x) orow[a] = 0.0f;
    return;
  }
  for (int a = threadIdx.x; a < Ta; a += blockDim.x) {
    float acc = 0.0f;
    for (int j = 0; j < n_heads; ++j) {
      const float* wr = w + (((int64_t)b * n_heads + j) * t_pad + t) * Ta;
      const float* mr = mean + ((int64_t)b * n_heads + j) * Ta;
      const float* sr = rstd + ((int64_t)b * n_heads + j) * Ta;
      float z[7];
#pragma unroll
      for (int o = 0; o < 7; ++o) {
        int i = a + o - 3;
        if (Ta > 3) {
          if (i < 0) i = -i;
          if (i >= Ta) i = 2 * (Ta - 1) - i;
        } else {
          i = a;                                  // too narrow to filter (dtw_align.py:68-69)
        }
        z[o] = (wr[i] - mr[i]) * sr[i];
      }
      acc += Ta > 3 ? median7(z[0], z[1], z[2], z[3], z[4], z[5], z[6]) : z[3];
    }
    orow[a] = acc / (float)n_heads;
  }
}

// ---------------------------------------------------------------------------
// Dynamic time warping of one chunk per CTA.  x[i][j] = -mat[row0 + i][j] inside the row's allowed
// column range, +inf outside.  Thread i owns text row i and walks it left to right, one anti-diagonal
// per step; the three live diagonals sit in shared memory, the chosen predecessor of every cell in a
// 2-bit trace (rows of ceil(M / 4) bytes, written only by the row's own thread).  Ties resolve
// diagonal, then up (text), then left (time), as in the reference.  Thread 0 walks the trace back.
// Outputs: text_idx / time_idx [path_cap] (forward order) and the path length.
// Dynamic shared memory: 3 * (N + 1) floats + N * ceil(M / 4) bytes + 2 * path ints are not needed at
// once: the path is written to global memory in reverse and turned round by all threads.
// ---------------------------------------------------------------------------
struct DtwParams {
  const float* mat; int64_t chunk_stride, ld;
  const int* row0; const int* n_rows; const int* n_cols;
  const int* col_lo; const int* col_hi; int limit_stride;     // nullptr: no limits
  int max_rows, max_cols, path_cap;
  int* text_idx; int* time_idx; int* path_len;
  DevStatus* status;
};

__global__ void __launch_bounds__(512) dtw_kernel(DtwParams p) {
  extern __shared__ __align__(16) uint8_t dtw_smem[];
  const int b = blockIdx.x;
  const int N = min(max(p.n_rows[b], 0), p.max_rows), M = min(max(p.n_cols[b], 0), p.max_cols);
  int* tout = p.text_idx + (int64_t)b * p.path_cap;
  int* jout = p.time_idx + (int64_t)b * p.path_cap;
  // a chunk whose rows or columns would leave its slab of the matrix is refused, not read
  const bool bad = p.row0[b] < 0 || M > p.ld || (p.chunk_stride > 0 && (int64_t)(p.row0[b] + N) * p.ld > p.chunk_stride);
  if (N == 0 || M == 0 || bad) {
    if (threadIdx.x == 0) {
      p.path_len[b] = 0;
      if (bad && p.status) atomicCAS(&p.status->code, 0, WDZ_EINVAL);
    }
    return;
  }
  const int rowbytes = (M + 3) >> 2;
  float* diag = reinterpret_cast<float*>(dtw_smem);                      // 3 x (max_rows + 1)
  const int dstride = p.max_rows + 1;
  uint8_t* trace = dtw_smem + (size_t)3 * dstride * sizeof(float);       // N x rowbytes
  const int i = threadIdx.x;                                             // text row 1..N (0 = border)
  for (int o = threadIdx.x; o < N * rowbytes; o += blockDim.x) trace[o] = 0;
  for (int o = threadIdx.x; o < 3 * dstride; o += blockDim.x) diag[o] = INFINITY;
  __syncthreads();
  if (threadIdx.x == 0) diag[0] = 0.0f;                                  // diagonal 0: cost[0][0]
  const float* mrow = nullptr;
  int lo = 0, hi = M;
  if (i >= 1 && i <= N) {
    mrow = p.mat + (int64_t)b * p.chunk_stride + (int64_t)(p.row0[b] + i - 1) * p.ld;
    if (p.col_lo) {
      lo = max(p.col_lo[(int64_t)b * p.limit_stride + i - 1], 0);
      hi = min(p.col_hi[(int64_t)b * p.limit_stride + i - 1], M);
    }
  }
  // The row's costs come through a ring of three float4 (columns c .. c + 11): a thread reads its row left to
  // right, one cell per diagonal, and with all rows live the lines do not stay in L1, so each load is issued
  // eight or more diagonals before its first use.
  const bool vec_ok = (p.ld & 3) == 0 && (p.chunk_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(p.mat) & 15) == 0;
  auto load4 = [&](int c0) -> float4 {
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (mrow == nullptr || c0 >= M) return v;
    if (vec_ok && c0 + 3 < p.ld) return *reinterpret_cast<const float4*>(mrow + c0);
    v.x = mrow[c0];
    if (c0 + 1 < M) v.y = mrow[c0 + 1];
    if (c0 + 2 < M) v.z = mrow[c0 + 2];
    if (c0 + 3 < M) v.w = mrow[c0 + 3];
    return v;
  };
  float4 r0 = load4(0), r1 = load4(4), r2 = load4(8);
  // diagonal k holds cost[i][k - i]; buffers rotate: d0 = k-2, d1 = k-1, d2 = k
  float* d0 = diag; float* d1 = diag + dstride; float* d2 = diag + 2 * dstride;
  // diagonal 1: cost[0][1] and cost[1][0] are borders (inf), already in place
  __syncthreads();
  for (int k = 2; k <= N + M; ++k) {
    if (i <= N) {
      const int j = k - i;
      float v = INFINITY;                                                // borders: row 0 (k > 0), column 0
      if (i >= 1 && j >= 1 && j <= M) {
        const int c = j - 1;
        const float raw = (c & 3) == 0 ? r0.x : (c & 3) == 1 ? r0.y : (c & 3) == 2 ? r0.z : r0.w;
        const float x = (c >= lo && c < hi) ? -raw : INFINITY;
        const float c0 = d0[i - 1], c1 = d1[i - 1], c2 = d1[i];
        int tdir; float cmin;
        if (c0 <= c1 && c0 <= c2) { cmin = c0; tdir = 0; }
        else if (c1 <= c2) { cmin = c1; tdir = 1; }
        else { cmin = c2; tdir = 2; }
        v = x + cmin;
        trace[(i - 1) * rowbytes + (c >> 2)] |= (uint8_t)(tdir << ((c & 3) * 2));
        if ((c & 3) == 3) { r0 = r1; r1 = r2; r2 = load4(c + 9); }
      }
      if (i >= 1 ? (j >= 0 && j <= M) : true) d2[i] = v;
    }
    __syncthreads();
    float* tmp = d0; d0 = d1; d1 = d2; d2 = tmp;
  }
  // backtrace, written from the end of the output arrays
  __shared__ int s_len;
  if (threadIdx.x == 0) {
    int bi = N, bj = M, n = 0;
    while ((bi > 0 || bj > 0) && n < p.path_cap) {
      tout[p.path_cap - 1 - n] = bi - 1;
      jout[p.path_cap - 1 - n] = bj - 1;
      int tdir;
      if (bi == 0) tdir = 2;
      else if (bj == 0) tdir = 1;
      else tdir = (trace[(bi - 1) * rowbytes + ((bj - 1) >> 2)] >> (((bj - 1) & 3) * 2)) & 3;
      if (tdir == 0) { --bi; --bj; }
      else if (tdir == 1) --bi;
      else --bj;
      ++n;
    }
    s_len = n;
    p.path_len[b] = n;
  }
  __syncthreads();
  // move the path to the front (it was written at [path_cap - len, path_cap)); the ranges may overlap,
  // so go through registers in rounds
  const int len = s_len, off = p.path_cap - len;
  if (off > 0) {
    for (int base = 0; base < len; base += blockDim.x) {
      const int n = base + threadIdx.x;
      int a = 0, c = 0;
      if (n < len) { a = tout[off + n]; c = jout[off + n]; }
      __syncthreads();
      if (n < len) { tout[n] = a; jout[n] = c; }
      __syncthreads();
    }
  }
}

inline size_t dtw_smem_bytes(int max_rows, int max_cols) {
  return (size_t)3 * (max_rows + 1) * sizeof(float) + (size_t)max_rows * ((max_cols + 3) / 4);
}

}  // namespace wdz
