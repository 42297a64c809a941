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
                    const wdz_rule_desc* __restrict__ rules, const uint32_t* __restrict__ tables, int n_tables,
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
      rd.n_set = rd.n_clear = rd.n_pen = 0; rd.arg0 = rd.arg1 = 0; rd.or_table = rd.allow_table = 0;
    }
  }
  __syncthreads();
  if (rd.forced_id >= 0) {
    if (tid == 0) out[r] = rd.forced_id;
    return;
  }
  const float* lg = logits + (int64_t)(row_idx ? row_idx[r] : r) * ld;
  const int n_set = min(max(rd.n_set, 0), 6), n_clear = min(max(rd.n_clear, 0), 4);
  const int n_pen = apply_penalty ? min(max(rd.n_pen, 0), 10) : 0;
  const bool have_tables = tables != nullptr;
  // tables named by index: a name outside the bound tables reads as "no table" (base table: nothing allowed)
  const uint32_t* t_base = have_tables && rd.mode == WDZ_MODE_ALL_EXCEPT_TABLE && rd.arg0 >= 0 && rd.arg0 < n_tables
                               ? tables + (int64_t)rd.arg0 * words : nullptr;
  const uint32_t* t_or = have_tables && rd.or_table > 0 && rd.or_table < n_tables ? tables + (int64_t)rd.or_table * words : nullptr;
  const uint32_t* t_allow = have_tables && rd.allow_table > 0 && rd.allow_table < n_tables
                                ? tables + (int64_t)rd.allow_table * words : nullptr;

  float bv = -INFINITY;
  int bi = 0x7fffffff;
  bool nan_here = false;
  for (int v = tid; v < V; v += 1024) {
    bool blocked;
    if (rd.mode == WDZ_MODE_OR) blocked = false;
    else if (rd.mode == WDZ_MODE_ALL_EXCEPT_TABLE)
      blocked = !(t_base && ((t_base[v >> 5] >> (v & 31)) & 1u));
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
    if (t_or) blocked |= (t_or[v >> 5] >> (v & 31)) & 1u;
    if (t_allow) blocked |= !((t_allow[v >> 5] >> (v & 31)) & 1u);
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

// ---------------------------------------------------------------------------
// Token-level rule state on the device.  The timestamp-pair rules need only a
// few integers per slot (how many tokens, parity and value of the last
// timestamp, the last ten text tokens), so the per-step host round trip of the
// reference (classify on the host, upload masks, download ids;
// decoding.py:1098-1456, 1766) can be dropped for them: one kernel turns each
// active slot's state into its rule descriptor and input token, and after the
// argmax another absorbs the new token.  Several decode steps can then be
// queued back to back; the host only polls the states.
// ---------------------------------------------------------------------------
namespace wdz {

struct TsParams {
  int eot, ts_begin, ts_end;        // 50257, 50365, 51865 for the multilingual vocabulary
  int first_timing_max;             // first timestamp within this many 0.02 s steps
  int open_after_close_span;        // next opening timestamp within this many steps of the last closing one
  uint32_t bit_special, bit_timings;  // class-table bits of the special and of the timestamp tokens
};

struct TsState {
  int max_new, n_new, timing_count, last_timing, last_was_timing, n_recent, done, last_token;
  int recent[10];
  int pad[6];
};  // 96 bytes

__global__ void ts_reset_kernel(const int* __restrict__ slots, const int* __restrict__ max_new, int n,
                                TsState* __restrict__ st, int n_slots) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int s = slots[r];
  if (s < 0 || s >= n_slots) return;
  TsState z{};
  z.max_new = max_new[r];
  z.last_timing = -1;
  st[s] = z;
}

// rules[r] and tokens[r] for the row of slot slots[r] (slot < 0: padded row, forced token 0).
__global__ void ts_rules_kernel(const int* __restrict__ slots, int n, const TsState* __restrict__ st, int n_slots,
                                TsParams tp, wdz_rule_desc* __restrict__ rules, int* __restrict__ tokens) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  wdz_rule_desc d{};
  d.forced_id = -1;
  const int slot = slots[r];
  if (slot < 0 || slot >= n_slots) {
    d.forced_id = 0;
    rules[r] = d;
    tokens[r] = 0;
    return;
  }
  const TsState s = st[slot];
  tokens[r] = s.last_token;
  const int n_timings = tp.ts_end - tp.ts_begin + 1;
  if (s.done || s.n_new >= s.max_new) {
    d.forced_id = tp.eot;
  } else if (s.timing_count == 0) {
    d.mode = WDZ_MODE_ALL_EXCEPT_RANGE;
    d.arg0 = tp.ts_begin;
    d.arg1 = tp.ts_begin + tp.first_timing_max + 1;
  } else if (s.timing_count & 1) {
    if (s.last_was_timing) {
      d.table_bits = tp.bit_special | tp.bit_timings;          // a word must follow an opening timestamp
    } else {
      d.table_bits = tp.bit_special;                            // text, or a closing timestamp later than the opening one
      d.prefix_begin = tp.ts_begin;
      d.prefix_end = tp.ts_begin + s.last_timing + 1;
    }
    d.n_pen = s.n_recent;
    for (int i = 0; i < 10; ++i) d.pen_ids[i] = s.recent[i];
  } else if (s.last_timing >= n_timings - 1) {
    d.forced_id = tp.eot;
  } else {                                                      // between pairs: next opening timestamp, or EOT
    d.mode = WDZ_MODE_ALL_EXCEPT_RANGE;
    d.arg0 = tp.ts_begin + s.last_timing;
    d.arg1 = min(tp.ts_end + 1, d.arg0 + tp.open_after_close_span);
    d.n_clear = 1;
    d.clear_ids[0] = tp.eot;
  }
  rules[r] = d;
}

// Absorbs next[r] into the state of slot slots[r] and appends it to the slot's token log.
// A row whose slot finishes is dropped from the row list (slot := -1) so that the remaining steps
// queued by the same call skip it in every kernel.
__global__ void ts_update_kernel(int* __restrict__ slots, int n, const int* __restrict__ next,
                                 TsState* __restrict__ st, int n_slots, TsParams tp, int* __restrict__ tok_log,
                                 int log_stride) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int slot = slots[r];
  if (slot < 0 || slot >= n_slots) return;
  TsState s = st[slot];
  if (s.done) { slots[r] = -1; return; }
  const int tok = next[r];
  if (s.n_new < log_stride) tok_log[(int64_t)slot * log_stride + s.n_new] = tok;
  s.n_new += 1;
  s.last_token = tok;
  if (tok == tp.eot || tok < 0) {
    s.done = 1;
    slots[r] = -1;
  } else if (tok >= tp.ts_begin && tok <= tp.ts_end) {
    s.timing_count += 1;
    s.last_timing = tok - tp.ts_begin;
    s.last_was_timing = 1;
  } else {
    s.last_was_timing = 0;
    if (s.n_recent >= 10) {
      for (int i = 0; i < 9; ++i) s.recent[i] = s.recent[i + 1];
      s.recent[9] = tok;
    } else {
      s.recent[s.n_recent++] = tok;
    }
  }
  st[slot] = s;
}

}  // namespace wdz
