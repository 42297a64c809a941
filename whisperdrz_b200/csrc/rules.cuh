// Logit rules + greedy argmax: the device half of decode_batch
// (src/whisperdrz/decoding.py:1514-1777): per-row blocked set assembled from
// bitset class tables and a few ids / id ranges, additive -65504, repetition
// penalty on the recent-token set, argmax with the lowest id winning ties
// (torch.argmax semantics), and the Phase-4 re-argmax without penalty
// (decoding.py:2033-2067).  One block per row; the ~200 KB logit row is read
// once.
#pragma once
#include "common.cuh"
#include "../../include/wdz.h"

namespace wdz {

__global__ void __launch_bounds__(1024)
rules_argmax_kernel(const float* __restrict__ logits, int64_t ld, const int* __restrict__ row_idx,
                    const wdz_rule_desc* __restrict__ rules, const uint32_t* __restrict__ tables,
                    int words, int V, int apply_penalty, int* __restrict__ out, DevStatus* status) {
  pdl_trigger();
  pdl_wait();
  __shared__ wdz_rule_desc rd;
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  __shared__ int saw_nan;
  const int r = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    saw_nan = 0;
    if (rules) rd = rules[r];
    else {
      rd.forced_id = -1; rd.mode = WDZ_MODE_OR; rd.table_bits = 0; rd.prefix_begin = rd.prefix_end = 0;
      rd.n_set = rd.n_clear = rd.n_pen = 0; rd.arg0 = rd.arg1 = 0;
    }
  }
  __syncthreads();
  if (rd.forced_id >= 0) {
    if (tid == 0) out[r] = rd.forced_id;
    return;
  }
  const float* lg = logits + (int64_t)(row_idx ? row_idx[r] : r) * ld;
  const int n_set = min(max(rd.n_set, 0), 8), n_clear = min(max(rd.n_clear, 0), 4);
  const int n_pen = apply_penalty ? min(max(rd.n_pen, 0), 10) : 0;
  const bool have_tables = tables != nullptr;

  float bv = -INFINITY;
  int bi = 0x7fffffff;
  bool nan_here = false;
  for (int v = tid; v < V; v += 1024) {
    bool blocked;
    if (rd.mode == WDZ_MODE_OR) blocked = false;
    else if (rd.mode == WDZ_MODE_ALL_EXCEPT_TABLE)
      blocked = !(have_tables && ((tables[(int64_t)rd.arg0 * words + (v >> 5)] >> (v & 31)) & 1u));
    else if (rd.mode == WDZ_MODE_ALL_EXCEPT_RANGE) blocked = !(v >= rd.arg0 && v < rd.arg1);
    else blocked = true;
    if (have_tables) {
      uint32_t bits = rd.table_bits;
      while (bits) {
        const int t = __ffs(bits) - 1;
        bits &= bits - 1;
        blocked |= (tables[(int64_t)t * words + (v >> 5)] >> (v & 31)) & 1u;
      }
    }
    blocked |= (v >= rd.prefix_begin && v < rd.prefix_end);
    for (int i = 0; i < n_set; ++i) blocked |= (rd.set_ids[i] == v);
    for (int i = 0; i < n_clear; ++i) if (rd.clear_ids[i] == v) blocked = false;
    float x = lg[v];
    nan_here |= (x != x);
    x += blocked ? -65504.0f : 0.0f;
    bool pen = false;
    for (int i = 0; i < n_pen; ++i) pen |= (rd.pen_ids[i] == v);
    if (pen) x = x > 0.0f ? x / 1.2f : x * 1.2f;
    if (x > bv) { bv = x; bi = v; }   // ids ascend per thread: strict > keeps the lowest
  }
  if (nan_here) saw_nan = 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { best_v[tid >> 5] = bv; best_i[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    bv = best_v[tid]; bi = best_i[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (tid == 0) {
      if (saw_nan || bi == 0x7fffffff) {
        out[r] = -1;
        if (status) atomicCAS(&status->code, 0, WDZ_ENAN);
      } else {
        out[r] = bi;
      }
    }
  }
}

}  // namespace wdz
