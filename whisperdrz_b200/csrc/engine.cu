// libwdz.so: the engine behind the C ABI of include/wdz.h.
//
// The engine owns no device memory: weights, KV caches and tables are lent by
// the host (wdz_bind) and all scratch comes from one caller-provided workspace
// (wdz_set_workspace) carved up here.  Every entry point only enqueues
// kernels on the caller's stream.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/wdz.h"
#include "attention.cuh"
#include "common.cuh"
#include "elementwise.cuh"
#include "gemm_simt.cuh"
#include "gemv_mma.cuh"
#include "logmel.cuh"
#include "rules.cuh"
#include "align.cuh"
#ifdef WDZ_WITH_TC
#include "gemm_tc.cuh"
#include "gemm_tc2.cuh"
#include "attn_tc.cuh"
#endif

using namespace wdz;

#ifdef WDZ_WITH_TC
struct wdz_engine;
static int gemm_tc_init(wdz_engine* e);
static int gemm_tc_launch(wdz_engine* e, int epi, const GemmParams& p, cudaStream_t s);
static int gemm_tc_swap_launch(wdz_engine* e, int epi, const GemvMmaParams& p, cudaStream_t s);
static int attn_tc_launch(wdz_engine* e, const void* qkv, void* out, int B, int T, int d, int H, cudaStream_t s,
                          const int* lens = nullptr, bool causal = false);
static int attn_tc_chunks_launch(wdz_engine* e, const void* q, void* out, const void* cache_k, const void* cache_v,
                                 int64_t S, int n_keys, int layer, const int* chunk_lens, const int* chunk_slots,
                                 int n_chunks, int t_pad, bool causal, cudaStream_t s);
#endif

namespace {

struct Bound { const void* ptr; int64_t numel; };

struct LayerW {
  const void *ln1_w, *ln1_b, *qkv_w, *qkv_b, *out_w, *out_b;
  const void *lnx_w, *lnx_b, *xq_w, *xq_b, *xout_w, *xout_b;  // decoder cross-attention
  const void *ln2_w, *ln2_b, *fc1_w, *fc1_b, *fc2_w, *fc2_b;
};

}  // namespace

struct wdz_engine {
  wdz_config cfg{};
  std::string err;
  std::unordered_map<std::string, Bound> bound;
  bool finalized = false;
  int device = 0;
  int sm_count = 148;
  int max_pairs = 0;   // CTA pairs (clusters of two) of gemm_tc2_kernel the device runs at once; 0 = kernel unused
  size_t esz = 2;

  // resolved tensors
  const void *conv1_w = nullptr, *conv1_b = nullptr, *conv2_w = nullptr, *conv2_b = nullptr;
  const float* enc_pos = nullptr;
  const void *ln_post_w = nullptr, *ln_post_b = nullptr;
  std::vector<LayerW> enc, dec;
  const void *tok_emb = nullptr, *dec_pos = nullptr, *dec_ln_w = nullptr, *dec_ln_b = nullptr;
  const void *xkv_w = nullptr, *xkv_b = nullptr;
  void *self_k = nullptr, *self_v = nullptr, *cross_k = nullptr, *cross_v = nullptr;
  int* seq_lens = nullptr;
  const uint32_t* tables = nullptr;
  int n_tables = 0;
  MelTables mel{};

  // workspace
  char* ws = nullptr;
  size_t ws_bytes = 0;
  float* mel_raw = nullptr; int* clipmax = nullptr;
  void *col1 = nullptr, *h1p = nullptr, *xn = nullptr, *qkv = nullptr, *ao = nullptr, *hid = nullptr;
  float* x = nullptr;
  float *dx = nullptr, *dxn = nullptr, *dqkv = nullptr, *dao = nullptr, *dq = nullptr, *dh = nullptr;
  float *part_o = nullptr, *part_ml = nullptr, *logits = nullptr;
  int* att_counters = nullptr;   // [max_rows] arrival counters of the split decode attention, zero between launches
  int* dpos = nullptr;
  int* al_slots = nullptr;     // rows of a teacher-forced alignment pass
  int* al_pos = nullptr;
  AlignHeads al_heads{};       // (layer, head) pairs of wdz_align_configure
  int al_last_layer = -1;
  DevStatus* status = nullptr;
  int64_t part_entries = 0;
  int max_emit = 0;
  int last_emit = 0;  // logit rows held from the last forward
  long long launches = 0;  // kernels enqueued since creation
  bool stream_attn_ok = false;  // bulk-copy cross-attention kernel usable for this shape
  // decode step as a CUDA graph, one per padded row count; inputs and outputs are staged
  // through fixed workspace buffers so that a replay needs no re-capture
  int *g_tokens = nullptr, *g_slots = nullptr, *g_next = nullptr;
  wdz_rule_desc* g_rules = nullptr;
  struct StepGraph { cudaGraphExec_t exec; long long launches; };
  std::unordered_map<int, StepGraph> step_graphs;
  std::unordered_map<int, StepGraph> ts_graphs;     // same step with the rule state kept on the device
  TsState* ts_state = nullptr;                       // [n_slots]
  int* ts_log = nullptr;                             // [n_slots, max_tokens] generated tokens per slot
  TsParams ts_params{50257, 50365, 51865, 50, 100, 1u, 2u};
  static constexpr int gemv_max_rows = 16;   // up to this many rows the mma.sync weight-streaming kernel runs, above it tcgen05
  cudaStream_t cap_stream = nullptr;  // capture happens here (the caller's stream may be the legacy default stream)
  // A decode step of many rows runs its layers as two half-batches on two streams (forked and joined with events, also
  // under capture), so that one half's products fill the SMs and the time in which the other half's attention streams
  // the K/V caches; created with the workspace, never during a capture.
  cudaStream_t side_stream = nullptr;
  bool pdl_suppress = false;   // the next launches go out without programmatic dependent launch
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_phase = nullptr;

  // optional per-kernel timing (wdz_profile): event pairs around selected launches
  struct Span { cudaEvent_t a, b; int kind; double work; };
  bool profiling = false;
  std::vector<Span> spans;
  size_t spans_used = 0;
  int span_begin(int kind, double work, cudaStream_t s) {
    if (!profiling) return -1;
    if (spans_used == spans.size()) {
      if (spans.size() >= 65536) return -1;
      Span sp{};
      if (cudaEventCreate(&sp.a) != cudaSuccess || cudaEventCreate(&sp.b) != cudaSuccess) { cudaGetLastError(); return -1; }
      spans.push_back(sp);
    }
    Span& sp = spans[spans_used];
    sp.kind = kind; sp.work = work;
    cudaEventRecord(sp.a, s);
    return (int)spans_used++;
  }
  void span_end(int id, cudaStream_t s) { if (id >= 0) cudaEventRecord(spans[id].b, s); }

  int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    err = buf;
    return code;
  }
};

namespace {

#define WDZ_LAUNCH_CHECK(e, what)                                                   \
  do {                                                                              \
    (e)->launches += 1;                                                             \
    cudaError_t _c = cudaGetLastError();                                            \
    if (_c != cudaSuccess) return (e)->fail(WDZ_ECUDA, "%s: %s", what, cudaGetErrorString(_c)); \
  } while (0)

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }
constexpr int SW_MAX_ROWS = 512;   // token rows per launch of the operand-swapped decode product
constexpr int SPLIT_MIN_ROWS = 320;  // a decode step of at least this many rows runs as two half-batches on two streams

// Launch with the programmatic stream-serialization attribute (kernels that call pdl_wait()).
template <typename... KArgs, typename... Args>
void launch_pdl(wdz_engine* e, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = ((e->cfg.flags & WDZ_FLAG_NO_PDL) || e->pdl_suppress) ? 0 : 1;
  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

int64_t part_entries_for(const wdz_config& c) {
  int64_t a = 8ll * c.max_rows, b = 2048;
  return a > b ? a : b;
}

// Carves the workspace; with base == nullptr only measures.
size_t carve(wdz_engine* e, char* base) {
  const wdz_config& c = e->cfg;
  const size_t es = e->esz;
  size_t off = 0;
  auto take = [&](size_t bytes) -> char* {
    char* p = base ? base + off : nullptr;
    off += align_up(bytes);
    return p;
  };
  const int64_t B = c.max_clips, Ta = c.n_audio_ctx, da = c.n_audio_state, R = c.max_rows, dt = c.n_text_state;
  const int H = c.n_text_head;
  e->status = (DevStatus*)take(sizeof(DevStatus));
  e->mel_raw = (float*)take(sizeof(float) * B * c.n_mels * MEL_MAX_FRAMES);
  e->clipmax = (int*)take(sizeof(int) * B);
  e->col1 = take(es * B * 2 * Ta * 3 * c.n_mels);
  e->h1p = take(es * B * (2 * Ta + 2) * da);
  e->x = (float*)take(sizeof(float) * B * Ta * da);
  e->xn = take(es * B * Ta * da);
  e->qkv = take(es * B * Ta * 3 * da);
  e->ao = take(es * B * Ta * da);
  e->hid = take(es * B * Ta * 4 * da);
  e->dx = (float*)take(sizeof(float) * R * dt);
  e->dxn = (float*)take(sizeof(float) * R * dt);
  e->dqkv = (float*)take(sizeof(float) * R * 3 * dt);
  e->dao = (float*)take(sizeof(float) * R * dt);
  e->dq = (float*)take(sizeof(float) * R * dt);
  e->dh = (float*)take(sizeof(float) * R * 4 * dt);
  e->dpos = (int*)take(sizeof(int) * R);
  e->al_slots = (int*)take(sizeof(int) * R);
  e->al_pos = (int*)take(sizeof(int) * R);
  e->g_tokens = (int*)take(sizeof(int) * (R + 8));
  e->g_slots = (int*)take(sizeof(int) * (R + 8));
  e->g_next = (int*)take(sizeof(int) * (R + 8));
  e->g_rules = (wdz_rule_desc*)take(sizeof(wdz_rule_desc) * (R + 8));
  e->ts_state = (TsState*)take(sizeof(TsState) * c.n_slots);
  e->ts_log = (int*)take(sizeof(int) * (size_t)c.n_slots * c.max_tokens);
  e->part_entries = part_entries_for(c);
  e->part_o = (float*)take(sizeof(float) * e->part_entries * H * HD);
  e->part_ml = (float*)take(sizeof(float) * e->part_entries * H * 2);
  e->att_counters = (int*)take(sizeof(int) * R);
  e->max_emit = c.max_rows < c.n_slots ? c.max_rows : c.n_slots;
  if (e->max_emit < 1) e->max_emit = 1;
  e->logits = (float*)take(sizeof(float) * (int64_t)e->max_emit * c.n_vocab);
  return off;
}

// ---- GEMM dispatch ---------------------------------------------------------
template <typename TA, typename TW, typename TO>
int launch_gemm_tile(wdz_engine* e, int epi, const GemmParams& p, cudaStream_t s) {
  dim3 grid((p.N + 63) / 64, (p.M + 63) / 64);
  switch (epi) {
    case EPI_STORE: gemm_tile_kernel<TA, TW, TO, EPI_STORE><<<grid, 256, 0, s>>>(p); break;
    case EPI_GELU: gemm_tile_kernel<TA, TW, TO, EPI_GELU><<<grid, 256, 0, s>>>(p); break;
    case EPI_RESID: gemm_tile_kernel<TA, TW, TO, EPI_RESID><<<grid, 256, 0, s>>>(p); break;
    case EPI_GELU_POS: gemm_tile_kernel<TA, TW, TO, EPI_GELU_POS><<<grid, 256, 0, s>>>(p); break;
    case EPI_CROSS_KV: gemm_tile_kernel<TA, TW, TO, EPI_CROSS_KV><<<grid, 256, 0, s>>>(p); break;
    default: return e->fail(WDZ_EINVAL, "bad epilogue %d", epi);
  }
  WDZ_LAUNCH_CHECK(e, "gemm_tile");
  return WDZ_OK;
}

GemmParams dense_params(const void* A, int64_t lda, const void* W, const void* bias, void* C, int64_t ldc,
                        int M, int N, int K) {
  GemmParams p{};
  p.A = A; p.W = W; p.bias = bias; p.C = C;
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldc = ldc;
  p.a_rpb = M > 0 ? M : 1; p.a_bstride = 0; p.c_rpb = M > 0 ? M : 1; p.c_bstride = 0;
  return p;
}

// Encoder-side product (A and outputs in T).  The tensor-core kernel takes the
// bf16 case when it is compiled in and not disabled.
template <typename T>
int enc_gemm(wdz_engine* e, int epi, const GemmParams& p, cudaStream_t s) {
  const int sp = e->span_begin(WDZ_PROF_ENC_GEMM, 2.0 * p.M * p.N * p.K, s);
  int rc = 1;
#ifdef WDZ_WITH_TC
  if (sizeof(T) == 2 && !(e->cfg.flags & WDZ_FLAG_NO_TENSOR_CORE)) rc = gemm_tc_launch(e, epi, p, s);
#endif
  if (rc == 1) rc = launch_gemm_tile<T, T, T>(e, epi, p, s);  // 1 = shape not taken by the tensor-core kernel
  e->span_end(sp, s);
  return rc;
}

template <typename T, int EPI>
int launch_gemv(wdz_engine* e, const GemvParams& p, cudaStream_t s) {
  // few columns per warp when N is small so that every SM streams weights
  const int warps_needed_1 = p.N;
  if (warps_needed_1 <= 8 * 2 * e->sm_count * 2) {
    launch_pdl(e, gemv_rows_kernel<T, EPI, 1>, dim3((p.N + 7) / 8), dim3(256), 0, s, p);
  } else if (p.N <= 8 * 4 * e->sm_count * 4) {
    launch_pdl(e, gemv_rows_kernel<T, EPI, 2>, dim3((p.N + 15) / 16), dim3(256), 0, s, p);
  } else {
    launch_pdl(e, gemv_rows_kernel<T, EPI, 4>, dim3((p.N + 31) / 32), dim3(256), 0, s, p);
  }
  WDZ_LAUNCH_CHECK(e, "gemv_rows");
  return WDZ_OK;
}

// Decode-side product: x f32 [M, K] -> y f32 [M, N].
template <typename T>
int dec_gemm(wdz_engine* e, int epi, const float* x, int64_t ldx, const void* W, const void* bias,
             float* y, int64_t ldy, int M, int N, int K, const int* row_idx, cudaStream_t s) {
  const int sp = e->span_begin(W == e->tok_emb ? WDZ_PROF_LM_HEAD : WDZ_PROF_DEC_GEMM,
                               (double)N * K * sizeof(T), s);
  int rc;
  if (M <= 64 || row_idx) {
    GemvParams p{x, W, bias, y, M, N, K, ldx, ldy, row_idx};
    switch (epi) {
      case EPI_STORE: rc = launch_gemv<T, EPI_STORE>(e, p, s); break;
      case EPI_GELU: rc = launch_gemv<T, EPI_GELU>(e, p, s); break;
      case EPI_RESID: rc = launch_gemv<T, EPI_RESID>(e, p, s); break;
      default: rc = e->fail(WDZ_EINVAL, "bad decode epilogue %d", epi);
    }
  } else {
    GemmParams p = dense_params(x, ldx, W, bias, y, ldy, M, N, K);
    rc = launch_gemm_tile<float, T, float>(e, epi, p, s);
  }
  e->span_end(sp, s);
  return rc;
}

template <typename TP, typename TO>
int launch_ln(wdz_engine* e, const float* x, int64_t ldx, const int* row_idx, const void* g, const void* b,
              TO* y, int64_t ldy, int rows, int d, cudaStream_t s, float* zero = nullptr, int64_t ldz = 0, int nz = 0) {
  if (rows <= 0) return WDZ_OK;
  if (zero && (rows > 1024 || (nz & 3) || (ldz & 3))) return e->fail(WDZ_EINVAL, "layernorm: cannot clear %d x %d", rows, nz);
  if (rows <= 1024)   // few rows: a CTA per row (latency-bound); many rows: a warp per row (bandwidth-bound)
    launch_pdl(e, layernorm_row_kernel<TP, TO>, dim3(rows), dim3(128), 0, s, x, ldx, row_idx, (const TP*)g,
               (const TP*)b, y, ldy, rows, d, zero, ldz, nz);
  else
  launch_pdl(e, layernorm_kernel<TP, TO>, dim3((rows + 3) / 4), dim3(128), 0, s, x, ldx, row_idx, (const TP*)g, (const TP*)b, y, ldy, rows, d);
  WDZ_LAUNCH_CHECK(e, "layernorm");
  return WDZ_OK;
}

// ---- encoder ---------------------------------------------------------------
// qkv T [B * Ta, 3d] -> out T [B * Ta, d]; tcgen05 kernel for bf16, CUDA cores otherwise.
template <typename T>
int enc_attention(wdz_engine* e, const void* qkv, void* out, int B, int Ta, int d, int H, cudaStream_t s) {
  const int sp = e->span_begin(WDZ_PROF_ENC_ATTN, 4.0 * B * H * (double)Ta * Ta * HD, s);
  int rc = 1;
#ifdef WDZ_WITH_TC
  if (sizeof(T) == 2 && !(e->cfg.flags & WDZ_FLAG_NO_TENSOR_CORE)) rc = attn_tc_launch(e, qkv, out, B, Ta, d, H, s);
#endif
  if (rc == 1) {
    attn_enc_simt_kernel<T><<<dim3((Ta + 63) / 64, H, B), 256, attn_enc_simt_smem(), s>>>((const T*)qkv, (T*)out, Ta, d);
    rc = WDZ_OK;
    e->launches += 1;
  }
  e->span_end(sp, s);
  if (rc != WDZ_OK) return rc;
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return e->fail(WDZ_ECUDA, "attn_enc: %s", cudaGetErrorString(ce));
  return WDZ_OK;
}

template <typename T>
int encode_impl(wdz_engine* e, const float* mel, int B, void* xa_out, cudaStream_t s) {
  const wdz_config& c = e->cfg;
  const int Ta = c.n_audio_ctx, frames = 2 * Ta, d = c.n_audio_state, H = c.n_audio_head;
  const int M = B * Ta;
  int rc;
  // conv1 as a product over the tap-major im2col operand
  im2col_conv1_kernel<T><<<dim3((frames + 31) / 32, B), 256, sizeof(float) * c.n_mels * 35, s>>>(
      mel, (T*)e->col1, c.n_mels, frames);
  WDZ_LAUNCH_CHECK(e, "im2col");
  const int64_t h1_b = (int64_t)(frames + 2) * d;  // one zero row before and after each window
  zero_rows_kernel<T><<<B, 256, 0, s>>>((T*)e->h1p, h1_b, 0, d, B);
  zero_rows_kernel<T><<<B, 256, 0, s>>>((T*)e->h1p, h1_b, (int64_t)(frames + 1) * d, d, B);
  WDZ_LAUNCH_CHECK(e, "zero_rows");
  {
    GemmParams p = dense_params(e->col1, 3 * c.n_mels, e->conv1_w, e->conv1_b, (T*)e->h1p + d, d,
                                B * frames, d, 3 * c.n_mels);
    p.c_rpb = frames; p.c_bstride = h1_b;
    if ((rc = enc_gemm<T>(e, EPI_GELU, p, s))) return rc;
  }
  // conv2 (stride 2): row (b, t) of the operand is the contiguous span
  // h1p[b, 2t .. 2t+2, :] of the padded conv1 output, so no im2col is needed.
  {
    GemmParams p = dense_params(e->h1p, 2 * d, e->conv2_w, e->conv2_b, e->x, d, M, d, 3 * d);
    p.a_rpb = Ta; p.a_bstride = h1_b;
    p.pos = e->enc_pos;
    if ((rc = enc_gemm<T>(e, EPI_GELU_POS, p, s))) return rc;
  }
  for (int l = 0; l < c.n_audio_layer; ++l) {
    const LayerW& w = e->enc[l];
    if ((rc = launch_ln<T, T>(e, e->x, d, nullptr, w.ln1_w, w.ln1_b, (T*)e->xn, d, M, d, s))) return rc;
    if ((rc = enc_gemm<T>(e, EPI_STORE, dense_params(e->xn, d, w.qkv_w, w.qkv_b, e->qkv, 3 * d, M, 3 * d, d), s))) return rc;
    if ((rc = enc_attention<T>(e, e->qkv, e->ao, B, Ta, d, H, s))) return rc;
    if ((rc = enc_gemm<T>(e, EPI_RESID, dense_params(e->ao, d, w.out_w, w.out_b, e->x, d, M, d, d), s))) return rc;
    if ((rc = launch_ln<T, T>(e, e->x, d, nullptr, w.ln2_w, w.ln2_b, (T*)e->xn, d, M, d, s))) return rc;
    if ((rc = enc_gemm<T>(e, EPI_GELU, dense_params(e->xn, d, w.fc1_w, w.fc1_b, e->hid, 4 * d, M, 4 * d, d), s))) return rc;
    if ((rc = enc_gemm<T>(e, EPI_RESID, dense_params(e->hid, 4 * d, w.fc2_w, w.fc2_b, e->x, d, M, d, 4 * d), s))) return rc;
  }
  return launch_ln<T, T>(e, e->x, d, nullptr, e->ln_post_w, e->ln_post_b, (T*)xa_out, d, M, d, s);
}

template <typename T>
int cross_kv_impl(wdz_engine* e, const void* xa, const int* slot_ids, int B, cudaStream_t s) {
  const wdz_config& c = e->cfg;
  const int d = c.n_text_state;
  GemmParams p = dense_params(xa, c.n_audio_state, e->xkv_w, e->xkv_b, nullptr, 0, B * c.n_audio_ctx,
                              c.n_text_layer * 2 * d, c.n_audio_state);
  p.cache_k = e->cross_k; p.cache_v = e->cross_v; p.slot_ids = slot_ids;
  p.n_slots = c.n_slots; p.T = c.n_audio_ctx; p.d = d;
  return enc_gemm<T>(e, EPI_CROSS_KV, p, s);
}

// ---- decoder ---------------------------------------------------------------
template <typename T>
int attn_dec_launch(wdz_engine* e, AttnDecParams p, int rows, int max_len, bool cross, cudaStream_t s, int sm_cap = 0,
                    int64_t part_cap = 0) {
  const int H = e->cfg.n_text_head;
  const bool stream = e->stream_attn_ok;
  // sm_cap > 0: a half-batch of a split step - walk the items with at most sm_cap CTAs and leave the other SMs to the
  // other half's products; part_cap: this half's share of the partial-result buffers
  const int sms = sm_cap > 0 && stream ? sm_cap : e->sm_count;
  const int64_t part_entries = part_cap > 0 ? part_cap : e->part_entries;
  int splits;
  // The streaming kernel walks (key range, row) items.  With few rows one persistent CTA per SM takes several items
  // and keeps its ring running across them (a 32-row step has only a wave or two of items, and every fresh CTA pays
  // the ring's start); with many rows one CTA per item does better, because a finished CTA's successor starts on
  // the hardware's own schedule while an item change inside a CTA stalls its head warps on the next query.
  const bool persistent = stream && (rows < 128 || sm_cap > 0);
  if (stream && !cross) {
    // lengths are only known on the device: fixed ranges, items past a row's length are skipped
    p.chunk = rows < 128 ? 64 : 128;
  } else if (stream) {
    // pick the split count whose items fill the SMs most evenly (whole waves of CTAs, or equal shares per CTA)
    int best = 1;
    double best_util = 0.0;
    for (int c = 1; c <= (rows <= 4 ? 46 : 24) && (int64_t)rows * c <= part_entries && max_len / c >= 32; ++c) {
      const int items = rows * c, per_cta = (items + sms - 1) / sms;
      const double util = (double)items / ((double)per_cta * sms);
      if (util > best_util + 0.03) { best_util = util; best = c; }
    }
    p.chunk = (max_len + best - 1) / best;
  } else if (cross) {
    splits = (3 * e->sm_count + rows - 1) / rows;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    p.chunk = ((max_len + splits - 1) / splits + 7) / 8 * 8;
  } else {
    p.chunk = 64;
  }
  splits = (max_len + p.chunk - 1) / p.chunk;
  if ((int64_t)rows * splits > part_entries)
    return e->fail(WDZ_ECAPACITY, "attention partials: %d rows x %d splits exceed the workspace", rows, splits);
  p.max_splits = splits;
  const int sp = e->span_begin(cross ? WDZ_PROF_CROSS_ATTN : WDZ_PROF_SELF_ATTN,
                               cross ? 2.0 * rows * max_len * p.d * sizeof(T) : 0.0, s);
  if (stream) {
    if (!p.counters) p.counters = e->att_counters;   // the last item of a row merges the row: no combine launch
    p.rows = rows;
    p.split_major = persistent ? 1 : 0;
    const int items = splits * rows;
    launch_pdl(e, attn_dec_stream_kernel<T>, dim3(persistent && items > sms ? sms : items), dim3((H + 1) * 32),
               attn_dec_stream_smem<T>(p.d), s, p, e->status);
    e->span_end(sp, s);
    WDZ_LAUNCH_CHECK(e, "attn_dec_stream");
    return WDZ_OK;
  } else {
    int hpc = 1;  // heads per CTA: the largest divisor of H up to 5, so that several CTAs share an SM
    for (int c = 2; c <= 5; ++c) if (H % c == 0) hpc = c;
    launch_pdl(e, attn_dec_kernel<T>, dim3(splits, rows, H / hpc), dim3(hpc * 32), 0, s, p);
  }
  e->span_end(sp, s);
  launch_pdl(e, attn_dec_combine_kernel<T>, dim3(rows), dim3(H * 32), 0, s, p);
  e->launches += 1;
  WDZ_LAUNCH_CHECK(e, "attn_dec");
  return WDZ_OK;
}

// bf16 decode product on the tensor cores (x bf16 [M, K], W bf16 [N, K]).
template <int EPI, bool OUT_BF16>
int launch_gemv_mma(wdz_engine* e, const GemvMmaParams& p, cudaStream_t s) {
  const int sp = e->span_begin(p.W == e->tok_emb ? WDZ_PROF_LM_HEAD : WDZ_PROF_DEC_GEMM, 2.0 * p.N * p.K, s);
  int rc = 1;
#ifdef WDZ_WITH_TC
  if (p.M > e->gemv_max_rows && !(e->cfg.flags & WDZ_FLAG_NO_TENSOR_CORE)) {
    // the operand-swapped tcgen05 kernel takes up to SW_MAX_ROWS rows per launch, in row tiles of at most 256
    for (int m0 = 0; m0 < p.M; m0 += SW_MAX_ROWS) {
      GemvMmaParams q = p;
      q.M = p.M - m0 < SW_MAX_ROWS ? p.M - m0 : SW_MAX_ROWS;
      q.x = p.x + (int64_t)m0 * p.ldx;
      q.y = OUT_BF16 ? (void*)((bf16*)p.y + (int64_t)m0 * p.ldy) : (void*)((float*)p.y + (int64_t)m0 * p.ldy);
      if (p.slots) q.slots = p.slots + m0;
      if (p.positions) q.positions = p.positions + m0;
      rc = gemm_tc_swap_launch(e, EPI, q, s);
      if (rc != WDZ_OK) break;   // 1 on the first chunk: shape not taken, nothing launched yet
    }
  }
#endif
  if (rc == 1) {
    launch_pdl(e, gemv_mma_kernel<EPI, OUT_BF16>, dim3((p.N + 15) / 16), dim3(256), 0, s, p);
    e->span_end(sp, s);
    WDZ_LAUNCH_CHECK(e, "gemv_mma");
    return WDZ_OK;
  }
  e->span_end(sp, s);
  return rc;
}

GemvMmaParams mma_params(const void* x, int64_t ldx, const void* W, const void* bias, void* y, int64_t ldy, int M,
                         int N, int K) {
  GemvMmaParams p{};
  p.x = (const bf16*)x; p.ldx = ldx; p.W = (const bf16*)W; p.bias = (const bf16*)bias; p.y = y; p.ldy = ldy;
  p.M = M; p.N = N; p.K = K;
  return p;
}

struct AlignCapture {   // teacher-forced alignment pass: keep the alignment heads' cross queries, stop after the last
  float* qcap; int64_t rows_total, row_base;
};

// tokens/slots/positions: device int32 [n].  Logits of the emit rows land in e->logits.
// Activations between kernels (LayerNorm output, attention output, MLP hidden)
// are stored in T; the residual stream, q/k/v of the new rows and the logits stay fp32.

template <typename T>
int forward_rows_impl(wdz_engine* e, const int* tokens, const int* slots, const int* positions, int n,
                      const int* emit_rows, int n_emit, cudaStream_t s, const AlignCapture* cap = nullptr) {
  constexpr bool kBf16 = sizeof(T) == 2;
  const wdz_config& c = e->cfg;
  const int d = c.n_text_state;
  int rc;
  T* xn = (T*)e->dxn;
  T* ao = (T*)e->dao;
  T* hid = (T*)e->dh;
  launch_pdl(e, embed_kernel<T>, dim3(n), dim3(256), 0, s, tokens, positions, (const T*)e->tok_emb, (const T*)e->dec_pos, e->dx, n, d,
                                     c.n_vocab, c.n_text_ctx);
  WDZ_LAUNCH_CHECK(e, "embed");
  // The layers over rows [r0, r0 + m) on stream st.  sm_cap / part_off / part_cap: see attn_dec_launch - a half-batch
  // of a split step walks its attention items with sm_cap CTAs and owns half of the partial-result buffers.
  auto run_layers = [&](int r0, int m, cudaStream_t st, int sm_cap, int64_t part_off, int64_t part_cap,
                        cudaEvent_t record_before_first_cross) -> int {
    const int* sl = slots + r0;
    const int* ps = positions + r0;
    float* dx = e->dx + (int64_t)r0 * d;
    T* xn_ = xn + (int64_t)r0 * d;
    T* ao_ = ao + (int64_t)r0 * d;
    T* hid_ = hid + (int64_t)r0 * 4 * d;
    float* dqkv = e->dqkv + (int64_t)r0 * 3 * d;
    float* dq = e->dq + (int64_t)r0 * d;
    const int H = c.n_text_head;
    AttnDecParams ap{};
    ap.n_slots = c.n_slots; ap.d = d; ap.slots = sl;
    ap.part_o = e->part_o + part_off * H * HD; ap.part_ml = e->part_ml + part_off * H * 2; ap.out = ao_; ap.ldo = d;
    ap.counters = e->att_counters + r0;
    // y = epi(x W^T + b) with x in T; RESID accumulates into the fp32 residual stream
    // next_w / next_bytes: the weights the following product will stream; the small-row kernel (<= 16 rows) pulls a
    // share of them into L2 while it runs, the many-row tcgen05 kernel ignores them
    auto gemm = [&](int epi, const T* x, int64_t ldx, const void* W, const void* bias, void* y, int64_t ldy, int M,
                    int N, int K, const void* next_w = nullptr, size_t next_bytes = 0) -> int {
      if constexpr (kBf16) {
        GemvMmaParams p = mma_params(x, ldx, W, bias, y, ldy, M, N, K);
        p.next_w = next_w; p.next_bytes = next_bytes;
        switch (epi) {
          case EPI_STORE: return launch_gemv_mma<EPI_STORE, false>(e, p, st);
          case EPI_RESID: return launch_gemv_mma<EPI_RESID, false>(e, p, st);
          case EPI_GELU: return launch_gemv_mma<EPI_GELU, true>(e, p, st);
          default: return e->fail(WDZ_EINVAL, "bad decode epilogue %d", epi);
        }
      } else {
        return dec_gemm<T>(e, epi, (const float*)x, ldx, W, bias, (float*)y, ldy, M, N, K, nullptr, st);
      }
    };
    int rc;
    // In a split step the product that follows an attention kernel goes out WITHOUT programmatic dependent launch:
    // launched early, its CTAs would sit on the SMs the attention walk leaves free, waiting for that attention to
    // end - exactly the SMs the other half's products are meant to run on (measured: 6033 ms per benchmark step with
    // the early launch, 5510 without).
    const bool plain_after_attention = part_cap > 0;
    for (int l = 0; l < c.n_text_layer; ++l) {
      const LayerW& w = e->dec[l];
      const size_t wb = (size_t)d * d * sizeof(T);   // bytes of one d x d weight
      const void* after = l + 1 < c.n_text_layer ? e->dec[l + 1].qkv_w : e->tok_emb;
      const size_t after_bytes = l + 1 < c.n_text_layer ? 3 * wb : (size_t)32 << 20;   // a first slice of the LM head
      if ((rc = launch_ln<T, T>(e, dx, d, nullptr, w.ln1_w, w.ln1_b, xn_, d, m, d, st))) return rc;
      if constexpr (kBf16) {
        // fused QKV projection whose epilogue appends K and V to the slot cache
        GemvMmaParams p = mma_params(xn_, d, w.qkv_w, w.qkv_b, dqkv, 3 * d, m, 3 * d, d);
        p.cache_k = (bf16*)e->self_k; p.cache_v = (bf16*)e->self_v; p.slots = sl; p.positions = ps;
        p.layer = l; p.n_slots = c.n_slots; p.S = c.max_tokens; p.d = d;
        p.next_w = w.out_w; p.next_bytes = wb;
        if ((rc = launch_gemv_mma<EPI_QKV_CACHE, false>(e, p, st))) return rc;
      } else {
        if ((rc = gemm(EPI_STORE, xn_, d, w.qkv_w, w.qkv_b, dqkv, 3 * d, m, 3 * d, d))) return rc;
        launch_pdl(e, kv_append_kernel<T>, dim3(m), dim3(256), 0, st, dqkv, sl, ps, (T*)e->self_k, (T*)e->self_v, l, c.n_slots,
                                               c.max_tokens, d, m);
        WDZ_LAUNCH_CHECK(e, "kv_append");
      }
      ap.layer = l;
      ap.q = dqkv; ap.ldq = 3 * d; ap.cache_k = e->self_k; ap.cache_v = e->self_v; ap.S = c.max_tokens;
      ap.positions = ps; ap.fixed_len = 0;
      if ((rc = attn_dec_launch<T>(e, ap, m, c.max_tokens, false, st, sm_cap, part_cap))) return rc;
      e->pdl_suppress = plain_after_attention;
      rc = gemm(EPI_RESID, ao_, d, w.out_w, w.out_b, dx, d, m, d, d, w.xq_w, wb);
      e->pdl_suppress = false;
      if (rc) return rc;

      // The cross-attention query is a complete-sum product of only d features: as such it would stream its
      // weights through a tenth of the SMs.  Its LayerNorm clears the query buffer instead and the product runs as
      // K-split partial sums added into it, like the residual products.
      const bool split_q = kBf16 && m > e->gemv_max_rows && m <= 1024 && !(c.flags & WDZ_FLAG_NO_TENSOR_CORE);
      if ((rc = launch_ln<T, T>(e, dx, d, nullptr, w.lnx_w, w.lnx_b, xn_, d, m, d, st, split_q ? dq : nullptr, d, d))) return rc;
      if ((rc = gemm(split_q ? EPI_RESID : EPI_STORE, xn_, d, w.xq_w, w.xq_b, dq, d, m, d, d, w.xout_w, wb))) return rc;
      if (cap) {
        int here = 0;
        for (int j = 0; j < e->al_heads.n; ++j) here += e->al_heads.layer[j] == l;
        if (here > 0) {
          align_capture_kernel<float><<<m, 64 * here, 0, st>>>(dq, d, m, l, e->al_heads, cap->qcap, cap->rows_total, cap->row_base);
          e->launches += 1;
          WDZ_LAUNCH_CHECK(e, "align_capture");
        }
        if (l >= e->al_last_layer) return 1;   // later layers cannot change the captured queries
      }
      if (l == 0) {
        // the two halves of a split step start half a layer apart, so that one is in its products while the other
        // streams its cross K/V
        if (record_before_first_cross && cudaEventRecord(record_before_first_cross, st) != cudaSuccess) {
          cudaError_t ce = cudaGetLastError();
          return e->fail(WDZ_ECUDA, "event record: %s", cudaGetErrorString(ce));
        }
      }
      ap.q = dq; ap.ldq = d; ap.cache_k = e->cross_k; ap.cache_v = e->cross_v; ap.S = c.n_audio_ctx;
      ap.positions = nullptr; ap.fixed_len = c.n_audio_ctx;
      if ((rc = attn_dec_launch<T>(e, ap, m, c.n_audio_ctx, true, st, sm_cap, part_cap))) return rc;
      e->pdl_suppress = plain_after_attention;
      rc = gemm(EPI_RESID, ao_, d, w.xout_w, w.xout_b, dx, d, m, d, d, w.fc1_w, 4 * wb);
      e->pdl_suppress = false;
      if (rc) return rc;

      if ((rc = launch_ln<T, T>(e, dx, d, nullptr, w.ln2_w, w.ln2_b, xn_, d, m, d, st))) return rc;
      if ((rc = gemm(EPI_GELU, xn_, d, w.fc1_w, w.fc1_b, hid_, 4 * d, m, 4 * d, d, w.fc2_w, 4 * wb))) return rc;
      if ((rc = gemm(EPI_RESID, hid_, 4 * d, w.fc2_w, w.fc2_b, dx, d, m, d, 4 * d, after, after_bytes))) return rc;
    }
    return WDZ_OK;
  };

  // Many rows: two half-batches on two streams.  The decode step alternates between products (tensor cores, weights)
  // and attention (HBM, almost no arithmetic); with the halves half a layer apart one half's attention streams its
  // K/V while the other half's products run on the SMs the attention walk leaves free.
  const bool split = kBf16 && !cap && !e->profiling && e->side_stream && e->stream_attn_ok && n >= SPLIT_MIN_ROWS &&
                     !(c.flags & (WDZ_FLAG_NO_SPLIT_STEP | WDZ_FLAG_NO_TENSOR_CORE));
  if (!split) {
    rc = run_layers(0, n, s, 0, 0, 0, nullptr);
    if (rc == 1) return WDZ_OK;   // alignment capture complete
    if (rc) return rc;
  } else {
    const int na = ((n + 1) / 2 + 31) / 32 * 32, nb = n - na;   // n >= SPLIT_MIN_ROWS, so both halves have rows
    const int64_t half = e->part_entries / 2;
    // CTAs of a half's attention walk: about two thirds of the SMs (the rest stay free for the other half's products),
    // trimmed so that every CTA gets the same number of whole rows - 96 CTAs of two rows each for a 192-row half,
    // where 92 or 105 CTAs measured 5 % slower per benchmark step
    const int sm_share = e->sm_count - e->sm_count / 3;
    auto attn_ctas_for = [&](int m) {
      const int per_cta = (m + sm_share - 1) / sm_share;
      const int ctas = (m + per_cta - 1) / per_cta;
      return ctas >= sm_share - sm_share / 5 ? ctas : sm_share;
    };
    cudaStream_t s2 = e->side_stream;
    bool ok = cudaEventRecord(e->ev_fork, s) == cudaSuccess && cudaStreamWaitEvent(s2, e->ev_fork, 0) == cudaSuccess;
    if (ok) {
      // the second half waits until the first has reached its first cross-attention
      rc = run_layers(0, na, s, attn_ctas_for(na), 0, half, e->ev_phase);
      if (rc) return rc;
      ok = cudaStreamWaitEvent(s2, e->ev_phase, 0) == cudaSuccess;
    }
    if (ok) {
      rc = run_layers(na, nb, s2, attn_ctas_for(nb), half, half, nullptr);
      if (rc) return rc;
      ok = cudaEventRecord(e->ev_join, s2) == cudaSuccess && cudaStreamWaitEvent(s, e->ev_join, 0) == cudaSuccess;
    }
    if (!ok) {
      cudaError_t ce = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "split step fork/join: %s", cudaGetErrorString(ce));
    }
  }
  launch_pdl(e, bump_seqlens_kernel, dim3((n + 255) / 256), dim3(256), 0, s, slots, positions, e->seq_lens, n, c.n_slots);
  WDZ_LAUNCH_CHECK(e, "bump_seqlens");
  // final LayerNorm on the emit rows only, then the tied LM head (model.py:609-613)
  if ((rc = launch_ln<T, T>(e, e->dx, d, emit_rows, e->dec_ln_w, e->dec_ln_b, xn, d, n_emit, d, s))) return rc;
  if constexpr (kBf16) {
    GemvMmaParams p = mma_params(xn, d, e->tok_emb, nullptr, e->logits, c.n_vocab, n_emit, c.n_vocab, d);
    if ((rc = launch_gemv_mma<EPI_STORE, false>(e, p, s))) return rc;
  } else {
    if ((rc = dec_gemm<T>(e, EPI_STORE, (const float*)xn, d, e->tok_emb, nullptr, e->logits, c.n_vocab, n_emit, c.n_vocab,
                          d, nullptr, s)))
      return rc;
  }
  e->last_emit = n_emit;
  return WDZ_OK;
}

// Copies the caller's step inputs into the fixed staging buffers and pads the
// row count: padded rows carry slot -1 (every kernel skips them) and a forced
// token so that the rule kernel never looks at their logits.
__global__ void stage_step_kernel(const int* __restrict__ tokens, const int* __restrict__ slots,
                                  const wdz_rule_desc* __restrict__ rules, int n, int npad,
                                  int* __restrict__ g_tokens, int* __restrict__ g_slots,
                                  wdz_rule_desc* __restrict__ g_rules) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;   // one thread per 32-bit word of a rule
  const int r = i >> 5, w = i & 31;
  if (r >= npad) return;
  int* dst = reinterpret_cast<int*>(g_rules + r);
  if (r < n) {
    if (w == 0) { g_tokens[r] = tokens[r]; g_slots[r] = slots[r]; }
    dst[w] = rules ? reinterpret_cast<const int*>(rules + r)[w] : (w == 0 ? -1 : 0);
  } else {
    if (w == 0) { g_tokens[r] = 0; g_slots[r] = -1; }
    dst[w] = 0;   // forced_id = 0
  }
}

int check_ready(wdz_engine* e) {
  if (!e) return WDZ_EINVAL;
  if (!e->finalized) return e->fail(WDZ_ESTATE, "engine not finalized");
  if (!e->ws) return e->fail(WDZ_ENOMEM, "no workspace set");
  return WDZ_OK;
}

int rules_launch(wdz_engine* e, const float* logits, const int* row_idx, const wdz_rule_desc* rules, int n,
                 int penalty, int* out, cudaStream_t s) {
  if (n <= 0) return WDZ_OK;
  const int V = e->cfg.n_vocab;
  launch_pdl(e, rules_argmax_kernel, dim3(n), dim3(1024), 0, s, logits, V, row_idx, rules, e->tables, e->n_tables, (V + 31) / 32, V, penalty, out,
                                         e->status);
  WDZ_LAUNCH_CHECK(e, "rules_argmax");
  return WDZ_OK;
}

}  // namespace

#ifdef WDZ_WITH_TC
// Tensor-core path: returns WDZ_OK when launched, 1 when the shape is left to
// the CUDA-core kernel, a negative code on failure.
static int gemm_tc_init(wdz_engine* e) {
  if (!tc::encode_fn()) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return e->fail(WDZ_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    tc::encode_fn() = (tc::EncodeTiledFn)fn;
  }
  if (cudaFuncSetAttribute(tc::gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES) !=
      cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "gemm_tc smem attribute: %s", cudaGetErrorString(ce));
  }
  // CTA-pair kernel: how many pairs the device holds at once (0 leaves every product to the lone-CTA kernel)
  e->max_pairs = 0;
  if (!(e->cfg.flags & WDZ_FLAG_NO_CTA_PAIRS) &&
      cudaFuncSetAttribute(tc2::gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2::SMEM_BYTES) == cudaSuccess) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * e->sm_count); cfg.blockDim = dim3(tc2::THREADS); cfg.dynamicSmemBytes = tc2::SMEM_BYTES;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, tc2::gemm_tc2_kernel, &cfg) == cudaSuccess && n > 0)
      e->max_pairs = n < e->sm_count / 2 ? n : e->sm_count / 2;
  }
  cudaGetLastError();
  if (cudaFuncSetAttribute(atc::attn_enc_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, atc::SMEM_BYTES) !=
          cudaSuccess ||
      cudaFuncSetAttribute(atc::attn_enc_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, atc::SMEM_BYTES) !=
          cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "attn_enc_tc smem attribute: %s", cudaGetErrorString(ce));
  }
  if (cudaFuncSetAttribute(tc::gemm_tc_swap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SW_SMEM_BYTES) !=
      cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "gemm_tc_swap smem attribute: %s", cudaGetErrorString(ce));
  }
  return WDZ_OK;
}

static int attn_tc_launch(wdz_engine* e, const void* qkv, void* out, int B, int T, int d, int H, cudaStream_t s,
                          const int* lens, bool causal) {
  if (((uintptr_t)qkv | (uintptr_t)out) & 15 || d % 8) return 1;
  CUtensorMap mq;
  if (!tc::make_map(&mq, qkv, (uint64_t)3 * d, (uint64_t)T, (uint64_t)B, (uint64_t)3 * d * 2, (uint64_t)T * 3 * d * 2,
                    128, 3))
    return 1;
  atc::AttnTcParams p{};
  p.out = (bf16*)out; p.out_rows = T; p.d = d; p.Tq = T; p.Tk = T;
  p.q_col0 = 0; p.k_col0 = d; p.v_col0 = 2 * d;
  p.lens = lens; p.causal = causal ? 1 : 0; p.one_map = 1;
  p.status = e->status;
  if (lens || causal)
    atc::attn_enc_tc_kernel<true><<<dim3((T + atc::QT - 1) / atc::QT, H, B), 192, atc::SMEM_BYTES, s>>>(mq, mq, mq, p);
  else
    atc::attn_enc_tc_kernel<false><<<dim3((T + atc::QT - 1) / atc::QT, H, B), 192, atc::SMEM_BYTES, s>>>(mq, mq, mq, p);
  e->launches += 1;
  return WDZ_OK;
}

// Teacher-forced pass: the t_pad query rows of each chunk (bf16 [chunks * t_pad, d]) against the cache rows of
// the chunk's slot in layer `layer`; cache [layers * slots, S, d].  Causal = self-attention over the chunk's own
// rows, else all n_keys cross keys.
static int attn_tc_chunks_launch(wdz_engine* e, const void* q, void* out, const void* cache_k, const void* cache_v,
                                 int64_t S, int n_keys, int layer, const int* chunk_lens, const int* chunk_slots,
                                 int n_chunks, int t_pad, bool causal, cudaStream_t s) {
  const wdz_config& c = e->cfg;
  const int d = c.n_text_state, H = c.n_text_head;
  if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache_k | (uintptr_t)cache_v) & 15 || d % 8) return 1;
  CUtensorMap mq, mk, mv;
  const uint64_t zs = (uint64_t)c.n_text_layer * c.n_slots;
  if (!tc::make_map(&mq, q, (uint64_t)d, (uint64_t)t_pad, (uint64_t)n_chunks, (uint64_t)d * 2, (uint64_t)t_pad * d * 2, 128, 3) ||
      !tc::make_map(&mk, cache_k, (uint64_t)d, (uint64_t)S, zs, (uint64_t)d * 2, (uint64_t)S * d * 2, 128, 3) ||
      !tc::make_map(&mv, cache_v, (uint64_t)d, (uint64_t)S, zs, (uint64_t)d * 2, (uint64_t)S * d * 2, 128, 3))
    return 1;
  atc::AttnTcParams p{};
  p.out = (bf16*)out; p.out_rows = t_pad; p.d = d; p.Tq = t_pad; p.Tk = n_keys;
  p.lens = chunk_lens; p.kv_z = chunk_slots; p.kv_z_base = layer * c.n_slots; p.kv_z_limit = c.n_slots;
  p.causal = causal ? 1 : 0;
  p.status = e->status;
  atc::attn_enc_tc_kernel<true><<<dim3((t_pad + atc::QT - 1) / atc::QT, H, n_chunks), 192, atc::SMEM_BYTES, s>>>(mq, mk, mv, p);
  e->launches += 1;
  return WDZ_OK;
}

// Decode-shaped product through the operand-swapped tcgen05 kernel.  Returns 1
// when the shape is left to the mma.sync kernel.
static int gemm_tc_swap_launch(wdz_engine* e, int epi, const GemvMmaParams& g, cudaStream_t s) {
  if (g.M < 1 || g.M > SW_MAX_ROWS || g.K % tc::BK) return 1;
  if ((((uintptr_t)g.x | (uintptr_t)g.W) & 15) || (g.ldx * 2) % 16) return 1;
  tc::TcSwapParams p{};
  p.bias = g.bias; p.y = g.y; p.ldy = g.ldy; p.M = g.M; p.N = g.N; p.K = g.K;
  // Row tile and K split.  A CTA takes in one 64-wide k-block of operands in 0.4 us (32 rows) to 0.8 us (256
  // rows) and all CTAs together about 6 TB/s, so the work is cut to cover the SMs in ONE wave:
  //  - complete sums (no K split): the smallest row tile whose CTAs still fit one wave;
  //  - residual sums (K split, red.global.add): a single row tile when K is long (operand bytes dominate),
  //    else 64- or 128-row tiles, and as many K splits as fill the wave.
  const int mpad_all = (g.M + 31) / 32 * 32;
  const int tiles = (g.N + tc::BM - 1) / tc::BM;
  p.kblocks = g.K / tc::BK;
  int row_tile = mpad_all;
  if (epi == EPI_RESID) {
    if (p.kblocks < 64) row_tile = std::min(mpad_all, g.M <= 128 ? 64 : 128);
  } else {
    for (int rt = 32; rt < mpad_all; rt *= 2)
      if (tiles * ((g.M + rt - 1) / rt) <= e->sm_count) { row_tile = rt; break; }
  }
  if (row_tile > 256) row_tile = 256;   // a row tile is the MMA N dimension and one accumulator of TMEM columns
  p.mpad = row_tile;
  const int row_tiles = (g.M + row_tile - 1) / row_tile;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.mpad) p.tmem_cols <<= 1;
  int ksplit = 1;
  if (epi == EPI_RESID) {
    ksplit = e->sm_count / (tiles * row_tiles);
    if (ksplit > p.kblocks) ksplit = p.kblocks;
    if (ksplit < 1) ksplit = 1;
  }
  p.kb_per_split = (p.kblocks + ksplit - 1) / ksplit;
  ksplit = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;
  p.epi = epi == EPI_QKV_CACHE ? tc::EPI_SW_QKV_CACHE : epi;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.mpad >> 3) << 17) | ((uint32_t)(tc::BM >> 4) << 24);
  p.cache_k = g.cache_k; p.cache_v = g.cache_v; p.slots = g.slots; p.positions = g.positions;
  p.layer = g.layer; p.n_slots = g.n_slots; p.S = g.S; p.d = g.d;
  p.status = e->status;
  CUtensorMap mw, mx;
  if (!tc::make_map(&mw, g.W, (uint64_t)g.K, (uint64_t)g.N, 1, (uint64_t)g.K * 2, (uint64_t)g.K * 2 * g.N, (uint32_t)tc::BM, 2))
    return 1;
  if (!tc::make_map(&mx, g.x, (uint64_t)g.K, (uint64_t)g.M, 1, (uint64_t)g.ldx * 2, (uint64_t)g.ldx * 2 * g.M,
                    (uint32_t)p.mpad, 2))
    return 1;
  launch_pdl(e, tc::gemm_tc_swap_kernel, dim3(tiles, ksplit, row_tiles), dim3(tc::SW_THREADS),
             (size_t)tc::sw_smem_bytes(row_tile), s, mw, mx, p);
  WDZ_LAUNCH_CHECK(e, "gemm_tc_swap");
  return WDZ_OK;
}

static int gemm_tc_launch(wdz_engine* e, int epi, const GemmParams& p, cudaStream_t s) {
  if (p.N % tc::BN || p.K % tc::BK || p.M < 1) return 1;
  if (((uintptr_t)p.A | (uintptr_t)p.W) & 15) return 1;
  if ((p.lda * 2) % 16 || (p.a_bstride * 2) % 16) return 1;
  if (epi != EPI_CROSS_KV && ((uintptr_t)p.C & 15)) return 1;
  if (epi != EPI_CROSS_KV && (p.ldc % 8 || p.c_bstride % 8)) return 1;
  if (epi == EPI_CROSS_KV && p.d % 32) return 1;
  tc::TcParams tp{};
  tp.g = p;
  tp.epi = epi;
  tp.status = e->status;
  const int rpb = p.a_rpb;
  tp.batches = (p.M + rpb - 1) / rpb;
  // 256-row tiles on CTA pairs wherever a batch has more rows than one CTA's 128
  const bool pairs = e->max_pairs > 0 && (rpb < p.M ? rpb : p.M) > tc::BM;
  if (pairs) {
    tp.tiles_m_per_batch = (rpb + tc2::PAIR_M - 1) / tc2::PAIR_M;
    tp.tiles_n = p.N / tc2::BN;
    tp.total_tiles = tp.batches * tp.tiles_m_per_batch * tp.tiles_n;
    tp.kblocks = p.K / tc::BK;
    CUtensorMap ma, mw;
    const uint64_t s1 = (uint64_t)p.lda * 2;
    const uint64_t s2 = tp.batches > 1 ? (uint64_t)p.a_bstride * 2 : s1 * (uint64_t)rpb;
    const uint64_t rows_last = tp.batches > 1 ? (uint64_t)rpb : (uint64_t)p.M;
    if (!tc::make_map(&ma, p.A, (uint64_t)p.K, rows_last, (uint64_t)tp.batches, s1, s2, tc2::BM_CTA, 3)) return 1;
    if (!tc::make_map(&mw, p.W, (uint64_t)p.K, (uint64_t)p.N, 1, (uint64_t)p.K * 2, (uint64_t)p.K * 2 * p.N, tc2::BN_CTA, 2))
      return 1;
    const int n_pairs = tp.total_tiles < e->max_pairs ? tp.total_tiles : e->max_pairs;
    tc2::gemm_tc2_kernel<<<2 * n_pairs, tc2::THREADS, tc2::SMEM_BYTES, s>>>(ma, mw, tp);
    WDZ_LAUNCH_CHECK(e, "gemm_tc2");
    return WDZ_OK;
  }
  tp.tiles_m_per_batch = (rpb + tc::BM - 1) / tc::BM;
  tp.tiles_n = p.N / tc::BN;
  tp.total_tiles = tp.batches * tp.tiles_m_per_batch * tp.tiles_n;
  tp.kblocks = p.K / tc::BK;
  CUtensorMap ma, mw;
  const uint64_t s1 = (uint64_t)p.lda * 2;
  const uint64_t s2 = tp.batches > 1 ? (uint64_t)p.a_bstride * 2 : s1 * (uint64_t)rpb;
  const uint64_t rows_last = tp.batches > 1 ? (uint64_t)rpb : (uint64_t)p.M;
  if (!tc::make_map(&ma, p.A, (uint64_t)p.K, rows_last, (uint64_t)tp.batches, s1, s2, tc::BM, 3)) return 1;
  if (!tc::make_map(&mw, p.W, (uint64_t)p.K, (uint64_t)p.N, 1, (uint64_t)p.K * 2, (uint64_t)p.K * 2 * p.N, tc::BN, 2))
    return 1;
  const int grid = tp.total_tiles < e->sm_count ? tp.total_tiles : e->sm_count;
  tc::gemm_tc_kernel<<<grid, tc::THREADS, tc::SMEM_BYTES, s>>>(ma, mw, tp);
  WDZ_LAUNCH_CHECK(e, "gemm_tc");
  return WDZ_OK;
}
#endif

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

const char* wdz_version(void) { return "wdz 0.1 (sm_100a)"; }

int wdz_engine_create(const wdz_config* cfg, wdz_engine** out) {
  if (!cfg || !out) return WDZ_EINVAL;
  *out = nullptr;
  const wdz_config& c = *cfg;
  if (c.dtype != WDZ_F32 && c.dtype != WDZ_BF16) return WDZ_EINVAL;
  if (c.n_audio_state != c.n_audio_head * HD || c.n_text_state != c.n_text_head * HD) return WDZ_EINVAL;
  if (c.n_audio_head > 32 || c.n_text_head > 32 || c.n_mels > 160 || c.n_mels < 1) return WDZ_EINVAL;
  if (c.n_slots < 1 || c.max_tokens < 1 || c.max_clips < 1 || c.max_rows < 1) return WDZ_EINVAL;
  if (c.n_audio_layer < 1 || c.n_text_layer < 1 || c.n_vocab < 1 || c.max_tokens > c.n_text_ctx) return WDZ_EINVAL;
  wdz_engine* e = new wdz_engine();
  e->cfg = c;
  e->esz = c.dtype == WDZ_BF16 ? 2 : 4;
  e->enc.resize(c.n_audio_layer);
  e->dec.resize(c.n_text_layer);
  if (cudaGetDevice(&e->device) == cudaSuccess) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, e->device) == cudaSuccess && sms > 0)
      e->sm_count = sms;
  } else {
    cudaGetLastError();
  }
  *out = e;
  return WDZ_OK;
}

int wdz_engine_destroy(wdz_engine* e) {
  if (e) {
    for (auto& sp : e->spans) { cudaEventDestroy(sp.a); cudaEventDestroy(sp.b); }
    for (auto& g : e->step_graphs) cudaGraphExecDestroy(g.second.exec);
    for (auto& g : e->ts_graphs) cudaGraphExecDestroy(g.second.exec);
    if (e->cap_stream) cudaStreamDestroy(e->cap_stream);
    if (e->side_stream) cudaStreamDestroy(e->side_stream);
    if (e->ev_fork) cudaEventDestroy(e->ev_fork);
    if (e->ev_join) cudaEventDestroy(e->ev_join);
    if (e->ev_phase) cudaEventDestroy(e->ev_phase);
  }
  delete e;
  return WDZ_OK;
}

const char* wdz_last_error(const wdz_engine* e) { return e ? e->err.c_str() : "null engine"; }

int wdz_workspace_bytes(const wdz_engine* e, size_t* out_bytes) {
  if (!e || !out_bytes) return WDZ_EINVAL;
  wdz_engine tmp;
  tmp.cfg = e->cfg;
  tmp.esz = e->esz;
  *out_bytes = carve(&tmp, nullptr) + 256;
  return WDZ_OK;
}

int wdz_set_workspace(wdz_engine* e, void* dev, size_t bytes) {
  if (!e || !dev) return WDZ_EINVAL;
  size_t need = 0;
  wdz_workspace_bytes(e, &need);
  if (bytes < need) return e->fail(WDZ_ENOMEM, "workspace of %zu bytes, need %zu", bytes, need);
  char* base = (char*)align_up((size_t)dev);
  carve(e, base);
  e->ws = base;
  e->ws_bytes = bytes;
  if (cudaMemset(e->status, 0, sizeof(DevStatus)) != cudaSuccess ||
      cudaMemset(e->att_counters, 0, sizeof(int) * e->cfg.max_rows) != cudaSuccess) {
    cudaGetLastError();
    return e->fail(WDZ_ECUDA, "cannot clear the status word");
  }
  // second stream and events of the split decode step (host objects, no device memory); without them the step
  // simply runs as one batch
  if (!e->side_stream && e->cfg.max_rows >= SPLIT_MIN_ROWS && !(e->cfg.flags & WDZ_FLAG_NO_SPLIT_STEP)) {
    if (cudaStreamCreateWithFlags(&e->side_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->ev_join, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->ev_phase, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      if (e->side_stream) { cudaStreamDestroy(e->side_stream); e->side_stream = nullptr; }
    }
  }
  return WDZ_OK;
}

int wdz_bind(wdz_engine* e, const char* name, const void* dev, int64_t numel) {
  if (!e || !name || !dev || numel <= 0) return WDZ_EINVAL;
  e->bound[name] = Bound{dev, numel};
  e->finalized = false;
  return WDZ_OK;
}

int wdz_finalize(wdz_engine* e) {
  if (!e) return WDZ_EINVAL;
  const wdz_config& c = e->cfg;
  int rc = WDZ_OK;
  auto get = [&](const std::string& name, int64_t numel, bool optional = false) -> const void* {
    auto it = e->bound.find(name);
    if (it == e->bound.end()) {
      if (!optional && rc == WDZ_OK) rc = e->fail(WDZ_ESTATE, "tensor '%s' was never bound", name.c_str());
      return nullptr;
    }
    if (it->second.numel != numel) {
      if (rc == WDZ_OK)
        rc = e->fail(WDZ_EINVAL, "tensor '%s' has %lld elements, expected %lld", name.c_str(),
                     (long long)it->second.numel, (long long)numel);
      return nullptr;
    }
    return it->second.ptr;
  };
  const int64_t da = c.n_audio_state, dt = c.n_text_state;
  e->conv1_w = get("encoder.conv1.weight", da * 3 * c.n_mels);
  e->conv1_b = get("encoder.conv1.bias", da);
  e->conv2_w = get("encoder.conv2.weight", da * 3 * da);
  e->conv2_b = get("encoder.conv2.bias", da);
  e->enc_pos = (const float*)get("encoder.positional_embedding", (int64_t)c.n_audio_ctx * da);
  e->ln_post_w = get("encoder.ln_post.weight", da);
  e->ln_post_b = get("encoder.ln_post.bias", da);
  auto block = [&](const std::string& p, LayerW& w, int64_t d, bool cross) {
    w.ln1_w = get(p + ".attn_ln.weight", d); w.ln1_b = get(p + ".attn_ln.bias", d);
    w.qkv_w = get(p + ".attn.qkv.weight", 3 * d * d); w.qkv_b = get(p + ".attn.qkv.bias", 3 * d);
    w.out_w = get(p + ".attn.out.weight", d * d); w.out_b = get(p + ".attn.out.bias", d);
    if (cross) {
      w.lnx_w = get(p + ".cross_attn_ln.weight", d); w.lnx_b = get(p + ".cross_attn_ln.bias", d);
      w.xq_w = get(p + ".cross_attn.query.weight", d * d); w.xq_b = get(p + ".cross_attn.query.bias", d);
      w.xout_w = get(p + ".cross_attn.out.weight", d * d); w.xout_b = get(p + ".cross_attn.out.bias", d);
    }
    w.ln2_w = get(p + ".mlp_ln.weight", d); w.ln2_b = get(p + ".mlp_ln.bias", d);
    w.fc1_w = get(p + ".mlp.0.weight", 4 * d * d); w.fc1_b = get(p + ".mlp.0.bias", 4 * d);
    w.fc2_w = get(p + ".mlp.2.weight", 4 * d * d); w.fc2_b = get(p + ".mlp.2.bias", d);
  };
  for (int l = 0; l < c.n_audio_layer; ++l) block("encoder.blocks." + std::to_string(l), e->enc[l], da, false);
  for (int l = 0; l < c.n_text_layer; ++l) block("decoder.blocks." + std::to_string(l), e->dec[l], dt, true);
  e->tok_emb = get("decoder.token_embedding.weight", (int64_t)c.n_vocab * dt);
  e->dec_pos = get("decoder.positional_embedding", (int64_t)c.n_text_ctx * dt);
  e->dec_ln_w = get("decoder.ln.weight", dt);
  e->dec_ln_b = get("decoder.ln.bias", dt);
  e->xkv_w = get("decoder.cross_kv.weight", (int64_t)c.n_text_layer * 2 * dt * da);
  e->xkv_b = get("decoder.cross_kv.bias", (int64_t)c.n_text_layer * 2 * dt);
  const int64_t self_n = (int64_t)c.n_text_layer * c.n_slots * c.max_tokens * dt;
  const int64_t cross_n = (int64_t)c.n_text_layer * c.n_slots * c.n_audio_ctx * dt;
  e->self_k = (void*)get("cache.self_k", self_n);
  e->self_v = (void*)get("cache.self_v", self_n);
  e->cross_k = (void*)get("cache.cross_k", cross_n);
  e->cross_v = (void*)get("cache.cross_v", cross_n);
  e->seq_lens = (int*)get("cache.seq_lens", c.n_slots);
  {
    // class tables of the logit rules: any number of vocabulary bitsets, at least WDZ_MAX_TABLES
    const int64_t words = (c.n_vocab + 31) / 32;
    auto it = e->bound.find("rules.tables");
    e->tables = nullptr; e->n_tables = 0;
    if (it != e->bound.end()) {
      if (it->second.numel % words || it->second.numel < (int64_t)WDZ_MAX_TABLES * words) {
        if (rc == WDZ_OK)
          rc = e->fail(WDZ_EINVAL, "tensor 'rules.tables' has %lld elements, expected a multiple of %lld and at least %lld",
                       (long long)it->second.numel, (long long)words, (long long)(WDZ_MAX_TABLES * words));
      } else {
        e->tables = (const uint32_t*)it->second.ptr;
        e->n_tables = (int)(it->second.numel / words);
      }
    }
  }
  e->mel.twiddle = (const float2*)get("mel.twiddle", 2 * MEL_NFFT);
  e->mel.window = (const float*)get("mel.window", MEL_NFFT);
  e->mel.fb = (const float*)get("mel.fb", (int64_t)MEL_BINS * c.n_mels);
  e->mel.band_lo = (const int*)get("mel.band_lo", c.n_mels);
  e->mel.band_hi = (const int*)get("mel.band_hi", c.n_mels);
  if (rc != WDZ_OK) return rc;

  cudaError_t ce = cudaFuncSetAttribute(logmel_raw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)logmel_smem_bytes());
  if (ce == cudaSuccess)
    ce = cudaFuncSetAttribute(attn_enc_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)attn_enc_simt_smem());
  if (ce == cudaSuccess)
    ce = cudaFuncSetAttribute(attn_enc_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)attn_enc_simt_smem());
  if (ce != cudaSuccess) {
    cudaGetLastError();
    return e->fail(WDZ_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(ce));
  }
#ifdef WDZ_WITH_TC
  if ((rc = gemm_tc_init(e)) != WDZ_OK) return rc;
#endif
  {
    const size_t need = c.dtype == WDZ_BF16 ? attn_dec_stream_smem<bf16>(c.n_text_state)
                                            : attn_dec_stream_smem<float>(c.n_text_state);
    e->stream_attn_ok = c.n_text_head <= 20 && need <= 227 * 1024 && !(c.flags & WDZ_FLAG_NO_BULK_COPY);
    if (e->stream_attn_ok) {
      cudaError_t ce2 = c.dtype == WDZ_BF16
          ? cudaFuncSetAttribute(attn_dec_stream_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need)
          : cudaFuncSetAttribute(attn_dec_stream_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
      if (ce2 != cudaSuccess) {
        cudaGetLastError();
        return e->fail(WDZ_ECUDA, "attn_dec_stream smem attribute: %s", cudaGetErrorString(ce2));
      }
    }
  }
  if (cudaFuncSetAttribute(dtw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
    cudaError_t ce3 = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "dtw smem attribute: %s", cudaGetErrorString(ce3));
  }
  if (c.dtype == WDZ_BF16 && c.n_text_state % 256)
    return e->fail(WDZ_EINVAL, "the bf16 decoder needs n_text_state to be a multiple of 256 (got %d)", c.n_text_state);
  e->finalized = true;
  return WDZ_OK;
}

int wdz_device_status(wdz_engine* e, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  DevStatus h{};
  cudaStream_t st = (cudaStream_t)s;
  if (cudaMemcpyAsync(&h, e->status, sizeof h, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "status read: %s", cudaGetErrorString(ce));
  }
  if (h.code != 0) {
    cudaMemsetAsync(e->status, 0, sizeof(DevStatus), st);
    cudaMemsetAsync(e->att_counters, 0, sizeof(int) * e->cfg.max_rows, st);   // a kernel that gave up may have left counts behind
    return e->fail(h.code, "device reported status %d (detail %d)", h.code, h.detail);
  }
  return WDZ_OK;
}

int wdz_linear(wdz_engine* e, const void* x_dev, int M, int K, const void* w_dev, const void* bias_dev, int N,
               int gelu, void* y_dev, int cuda_cores_only, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!x_dev || !w_dev || !y_dev || M < 1 || N < 1 || K < 1) return e->fail(WDZ_EINVAL, "wdz_linear: bad argument");
  GemmParams p = dense_params(x_dev, K, w_dev, bias_dev, y_dev, N, M, N, K);
  const int epi = gelu ? EPI_GELU : EPI_STORE;
  cudaStream_t st = (cudaStream_t)s;
  if (e->cfg.dtype == WDZ_F32) return launch_gemm_tile<float, float, float>(e, epi, p, st);
  const int saved = e->cfg.flags;
  const int saved_pairs = e->max_pairs;
  if (cuda_cores_only == 1) e->cfg.flags |= WDZ_FLAG_NO_TENSOR_CORE;
  if (cuda_cores_only == 2) e->max_pairs = 0;
  rc = enc_gemm<bf16>(e, epi, p, st);
  e->cfg.flags = saved;
  e->max_pairs = saved_pairs;
  return rc;
}

int wdz_linear_rows(wdz_engine* e, const void* x_dev, int M, int K, const void* w_dev, const void* bias_dev, int N,
                    int accumulate, float* y_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!x_dev || !w_dev || !y_dev || M < 1 || N < 1 || K < 1) return e->fail(WDZ_EINVAL, "wdz_linear_rows: bad argument");
  cudaStream_t st = (cudaStream_t)s;
  if (e->cfg.dtype == WDZ_F32)
    return dec_gemm<float>(e, accumulate ? EPI_RESID : EPI_STORE, (const float*)x_dev, K, w_dev, bias_dev, y_dev, N, M, N,
                           K, nullptr, st);
  if (K % 256) return e->fail(WDZ_EINVAL, "wdz_linear_rows: bf16 needs K %% 256 == 0");
  GemvMmaParams p = mma_params(x_dev, K, w_dev, bias_dev, y_dev, N, M, N, K);
  return accumulate ? launch_gemv_mma<EPI_RESID, false>(e, p, st) : launch_gemv_mma<EPI_STORE, false>(e, p, st);
}

int wdz_encoder_attention(wdz_engine* e, const void* qkv_dev, int B, void* out_dev, int cuda_cores_only, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!qkv_dev || !out_dev || B < 1) return e->fail(WDZ_EINVAL, "wdz_encoder_attention: bad argument");
  const wdz_config& c = e->cfg;
  const int saved = e->cfg.flags;
  if (cuda_cores_only) e->cfg.flags |= WDZ_FLAG_NO_TENSOR_CORE;
  rc = c.dtype == WDZ_BF16
           ? enc_attention<bf16>(e, qkv_dev, out_dev, B, c.n_audio_ctx, c.n_audio_state, c.n_audio_head, (cudaStream_t)s)
           : enc_attention<float>(e, qkv_dev, out_dev, B, c.n_audio_ctx, c.n_audio_state, c.n_audio_head, (cudaStream_t)s);
  e->cfg.flags = saved;
  return rc;
}

int wdz_launch_count(const wdz_engine* e, int64_t* out) {
  if (!e || !out) return WDZ_EINVAL;
  *out = e->launches;
  return WDZ_OK;
}

int wdz_profile(wdz_engine* e, int enable) {
  if (!e) return WDZ_EINVAL;
  e->profiling = enable != 0;
  if (enable) e->spans_used = 0;
  return WDZ_OK;
}

int wdz_profile_read(wdz_engine* e, int kind, double* total_ms, int64_t* launches, double* work) {
  if (!e || !total_ms || !launches || !work) return WDZ_EINVAL;
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "profile read: %s", cudaGetErrorString(ce));
  }
  *total_ms = 0.0; *launches = 0; *work = 0.0;
  for (size_t i = 0; i < e->spans_used; ++i) {
    const wdz_engine::Span& sp = e->spans[i];
    if (sp.kind != kind) continue;
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, sp.a, sp.b) != cudaSuccess) { cudaGetLastError(); continue; }
    *total_ms += ms; *launches += 1; *work += sp.work;
  }
  return WDZ_OK;
}

int wdz_logmel(wdz_engine* e, const float* audio_dev, int64_t audio_stride, const int32_t* n_samples_dev,
               const int32_t* frame_offset_dev, int B, float* mel_out_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!audio_dev || !n_samples_dev || !mel_out_dev || B < 0) return e->fail(WDZ_EINVAL, "wdz_logmel: null argument");
  if (B == 0) return WDZ_OK;
  if (B > e->cfg.max_clips) return e->fail(WDZ_ECAPACITY, "wdz_logmel: %d clips > max_clips %d", B, e->cfg.max_clips);
  cudaStream_t st = (cudaStream_t)s;
  const int sp = e->span_begin(WDZ_PROF_LOGMEL, 0.0, st);
  logmel_init_max_kernel<<<(B + 255) / 256, 256, 0, st>>>(e->clipmax, B);
  logmel_raw_kernel<<<dim3((MEL_MAX_FRAMES + MEL_FT - 1) / MEL_FT, B), 256, logmel_smem_bytes(), st>>>(
      audio_dev, audio_stride, n_samples_dev, e->mel, e->cfg.n_mels, e->mel_raw, e->clipmax);
  logmel_finalize_kernel<<<dim3((MEL_MAX_FRAMES + 255) / 256, e->cfg.n_mels, B), 256, 0, st>>>(
      e->mel_raw, e->clipmax, n_samples_dev, frame_offset_dev, e->cfg.n_mels, mel_out_dev);
  e->span_end(sp, st);
  e->launches += 2;
  WDZ_LAUNCH_CHECK(e, "logmel");
  return WDZ_OK;
}

// ---- log-mel with built-in scratch -----------------------------------------
// The two intermediates of the front end (un-normalised log-mel of every frame
// and the per-clip maximum) normally live in the caller-provided workspace.
// This variant keeps them in a fixed array that is part of the library image,
// so it can serve hosts that have no workspace to give.  Every GPU that loads
// the library carries the array (about 6.1 MB) until the process exits.
#define WDZ_STATIC_MEL_FLOATS (WDZ_STATIC_MAX_CLIPS * WDZ_STATIC_MAX_MELS * MEL_MAX_FRAMES)
static __device__ __align__(256) float g_static_mel_scratch[WDZ_STATIC_MEL_FLOATS + 64];
static std::mutex g_static_mu;
static float* g_static_mel_ptr[64] = {};   // device address of the array, per device ordinal

int wdz_logmel_static(wdz_engine* e, const float* audio_dev, int64_t audio_stride, const int32_t* n_samples_dev,
                      const int32_t* frame_offset_dev, int B, float* mel_out_dev, wdz_stream s) {
  if (!e) return WDZ_EINVAL;
  if (!e->finalized) return e->fail(WDZ_ESTATE, "engine not finalized");
  if (!audio_dev || !n_samples_dev || !mel_out_dev || B < 0)
    return e->fail(WDZ_EINVAL, "wdz_logmel_static: null argument");
  if (B == 0) return WDZ_OK;
  if (B > WDZ_STATIC_MAX_CLIPS)
    return e->fail(WDZ_ECAPACITY, "wdz_logmel_static: %d clips, the built-in scratch holds at most %d", B,
                   WDZ_STATIC_MAX_CLIPS);
  if (e->cfg.n_mels > WDZ_STATIC_MAX_MELS)
    return e->fail(WDZ_ECAPACITY, "wdz_logmel_static: %d mel bins, the built-in scratch holds at most %d",
                   e->cfg.n_mels, WDZ_STATIC_MAX_MELS);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return e->fail(WDZ_ECUDA, "wdz_logmel_static: cannot tell the current device");
  }
  if (dev != e->device)
    return e->fail(WDZ_EINVAL, "wdz_logmel_static: device %d is current but the engine lives on %d", dev, e->device);
  float* scratch = nullptr;
  {
    // set-up, once per device: the array's name is only a handle on the host,
    // the kernels need its address in that device's memory
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_mel_ptr[dev]) {
      void* p = nullptr;
      cudaError_t ce = cudaGetSymbolAddress(&p, g_static_mel_scratch);
      if (ce != cudaSuccess || !p) {
        cudaGetLastError();
        return e->fail(WDZ_ECUDA, "wdz_logmel_static: cudaGetSymbolAddress: %s", cudaGetErrorString(ce));
      }
      g_static_mel_ptr[dev] = (float*)p;
    }
    scratch = g_static_mel_ptr[dev];
  }
  float* raw = scratch;
  int* clipmax = reinterpret_cast<int*>(scratch + WDZ_STATIC_MEL_FLOATS);
  cudaStream_t st = (cudaStream_t)s;
  // the per-clip maxima are the only state that must not survive from the previous call
  logmel_init_max_kernel<<<1, 64, 0, st>>>(clipmax, B);
  logmel_raw_kernel<<<dim3((MEL_MAX_FRAMES + MEL_FT - 1) / MEL_FT, B), 256, logmel_smem_bytes(), st>>>(
      audio_dev, audio_stride, n_samples_dev, e->mel, e->cfg.n_mels, raw, clipmax);
  logmel_finalize_kernel<<<dim3((MEL_MAX_FRAMES + 255) / 256, e->cfg.n_mels, B), 256, 0, st>>>(
      raw, clipmax, n_samples_dev, frame_offset_dev, e->cfg.n_mels, mel_out_dev);
  e->launches += 2;
  WDZ_LAUNCH_CHECK(e, "logmel_static");
  return WDZ_OK;
}

int wdz_encode(wdz_engine* e, const float* mel_dev, int B, void* xa_out_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!mel_dev || !xa_out_dev || B < 0) return e->fail(WDZ_EINVAL, "wdz_encode: null argument");
  if (B == 0) return WDZ_OK;
  if (B > e->cfg.max_clips) return e->fail(WDZ_ECAPACITY, "wdz_encode: %d clips > max_clips %d", B, e->cfg.max_clips);
  return e->cfg.dtype == WDZ_BF16 ? encode_impl<bf16>(e, mel_dev, B, xa_out_dev, (cudaStream_t)s)
                                  : encode_impl<float>(e, mel_dev, B, xa_out_dev, (cudaStream_t)s);
}

int wdz_cross_kv(wdz_engine* e, const void* xa_dev, const int32_t* slot_ids_dev, int B, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!xa_dev || !slot_ids_dev || B < 0) return e->fail(WDZ_EINVAL, "wdz_cross_kv: null argument");
  if (B == 0) return WDZ_OK;
  if (B > e->cfg.max_clips) return e->fail(WDZ_ECAPACITY, "wdz_cross_kv: %d windows > max_clips %d", B, e->cfg.max_clips);
  return e->cfg.dtype == WDZ_BF16 ? cross_kv_impl<bf16>(e, xa_dev, slot_ids_dev, B, (cudaStream_t)s)
                                  : cross_kv_impl<float>(e, xa_dev, slot_ids_dev, B, (cudaStream_t)s);
}

int wdz_slot_reset(wdz_engine* e, const int32_t* slot_ids_dev, int n, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!slot_ids_dev || n < 0) return e->fail(WDZ_EINVAL, "wdz_slot_reset: null argument");
  if (n == 0) return WDZ_OK;
  reset_seqlens_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)s>>>(slot_ids_dev, e->seq_lens, n, e->cfg.n_slots);
  WDZ_LAUNCH_CHECK(e, "slot_reset");
  return WDZ_OK;
}

int wdz_slot_seqlens(wdz_engine* e, int32_t* out_host, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!out_host) return e->fail(WDZ_EINVAL, "wdz_slot_seqlens: null argument");
  cudaStream_t st = (cudaStream_t)s;
  if (cudaMemcpyAsync(out_host, e->seq_lens, sizeof(int) * e->cfg.n_slots, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "seq_lens read: %s", cudaGetErrorString(ce));
  }
  return WDZ_OK;
}

int wdz_forward_rows(wdz_engine* e, const int32_t* tokens_dev, const int32_t* slot_ids_dev,
                     const int32_t* positions_dev, int n, const int32_t* emit_rows_dev, int n_emit,
                     float* logits_out_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!tokens_dev || !slot_ids_dev || !positions_dev || n < 0) return e->fail(WDZ_EINVAL, "wdz_forward_rows: null argument");
  if (n == 0) return WDZ_OK;
  if (n > e->cfg.max_rows) return e->fail(WDZ_ECAPACITY, "wdz_forward_rows: %d rows > max_rows %d", n, e->cfg.max_rows);
  if (!emit_rows_dev) n_emit = n;
  if (n_emit < 0 || n_emit > e->max_emit)
    return e->fail(WDZ_ECAPACITY, "wdz_forward_rows: %d logit rows > %d", n_emit, e->max_emit);
  cudaStream_t st = (cudaStream_t)s;
  rc = e->cfg.dtype == WDZ_BF16
           ? forward_rows_impl<bf16>(e, tokens_dev, slot_ids_dev, positions_dev, n, emit_rows_dev, n_emit, st)
           : forward_rows_impl<float>(e, tokens_dev, slot_ids_dev, positions_dev, n, emit_rows_dev, n_emit, st);
  if (rc) return rc;
  if (logits_out_dev && n_emit > 0) {
    if (cudaMemcpyAsync(logits_out_dev, e->logits, sizeof(float) * (size_t)n_emit * e->cfg.n_vocab,
                        cudaMemcpyDeviceToDevice, st) != cudaSuccess) {
      cudaError_t ce = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "logits copy: %s", cudaGetErrorString(ce));
    }
  }
  return WDZ_OK;
}

int wdz_prefill(wdz_engine* e, const void* xa_dev, const int32_t* window_slot_ids_dev, int B,
                const int32_t* tokens_dev, const int32_t* slot_ids_dev, const int32_t* positions_dev, int n,
                const int32_t* emit_rows_dev, int n_emit, float* logits_out_dev, wdz_stream s) {
  int rc = wdz_cross_kv(e, xa_dev, window_slot_ids_dev, B, s);
  if (rc) return rc;
  if ((rc = wdz_slot_reset(e, window_slot_ids_dev, B, s))) return rc;
  return wdz_forward_rows(e, tokens_dev, slot_ids_dev, positions_dev, n, emit_rows_dev, n_emit, logits_out_dev, s);
}

// The work of one decode step on fixed buffers: positions from the slot
// lengths, the forward over all rows, logit rules + argmax.
static int decode_step_body(wdz_engine* e, const int* tokens, const int* slots, const wdz_rule_desc* rules, int n,
                            int* next_out, cudaStream_t st) {
  launch_pdl(e, positions_from_seqlens_kernel, dim3((n + 255) / 256), dim3(256), 0, st, slots, e->seq_lens, e->dpos, n, e->cfg.n_slots);
  WDZ_LAUNCH_CHECK(e, "positions");
  int rc = wdz_forward_rows(e, tokens, slots, e->dpos, n, nullptr, n, nullptr, (wdz_stream)st);
  if (rc) return rc;
  return rules_launch(e, e->logits, nullptr, rules, n, 1, next_out, st);
}

int wdz_decode_step(wdz_engine* e, const int32_t* tokens_dev, const int32_t* slot_ids_dev, int n_active,
                    const wdz_rule_desc* rules_dev, int32_t* next_tokens_out_dev, float* logits_out_dev,
                    wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!tokens_dev || !slot_ids_dev || !next_tokens_out_dev || n_active < 0)
    return e->fail(WDZ_EINVAL, "wdz_decode_step: null argument");
  if (n_active == 0) return WDZ_OK;
  const int cap = e->cfg.max_rows < e->max_emit ? e->cfg.max_rows : e->max_emit;
  if (n_active > cap) return e->fail(WDZ_ECAPACITY, "wdz_decode_step: %d rows > capacity %d", n_active, cap);
  cudaStream_t st = (cudaStream_t)s;
  const bool use_graph = !(e->cfg.flags & WDZ_FLAG_NO_GRAPH) && !e->profiling;
  if (!use_graph) {
    if ((rc = decode_step_body(e, tokens_dev, slot_ids_dev, rules_dev, n_active, next_tokens_out_dev, st))) return rc;
  } else {
    int npad = (n_active + 7) / 8 * 8;
    if (npad > cap) npad = n_active;
    stage_step_kernel<<<(npad * 32 + 255) / 256, 256, 0, st>>>(tokens_dev, slot_ids_dev, rules_dev, n_active, npad,
                                                                 e->g_tokens, e->g_slots, e->g_rules);
    WDZ_LAUNCH_CHECK(e, "stage_step");
    auto it = e->step_graphs.find(npad);
    if (it == e->step_graphs.end()) {
      const long long before = e->launches;
      cudaGraph_t graph = nullptr;
      if (!e->cap_stream && cudaStreamCreateWithFlags(&e->cap_stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaError_t ce0 = cudaGetLastError();
        return e->fail(WDZ_ECUDA, "capture stream: %s", cudaGetErrorString(ce0));
      }
      if (cudaStreamBeginCapture(e->cap_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaError_t ce0 = cudaGetLastError();
        return e->fail(WDZ_ECUDA, "graph capture begin: %s", cudaGetErrorString(ce0));
      }
      rc = decode_step_body(e, e->g_tokens, e->g_slots, e->g_rules, npad, e->g_next, e->cap_stream);
      cudaError_t ce = cudaStreamEndCapture(e->cap_stream, &graph);
      if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
      if (ce != cudaSuccess || !graph) {
        cudaGetLastError();
        return e->fail(WDZ_ECUDA, "graph capture end: %s", cudaGetErrorString(ce));
      }
      wdz_engine::StepGraph g{};
      ce = cudaGraphInstantiate(&g.exec, graph, 0);
      cudaGraphDestroy(graph);
      if (ce != cudaSuccess) {
        cudaGetLastError();
        return e->fail(WDZ_ECUDA, "graph instantiate: %s", cudaGetErrorString(ce));
      }
      g.launches = e->launches - before;
      e->launches = before;
      it = e->step_graphs.emplace(npad, g).first;
    }
    if (cudaGraphLaunch(it->second.exec, st) != cudaSuccess) {
      cudaError_t ce = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "graph launch: %s", cudaGetErrorString(ce));
    }
    e->launches += it->second.launches;
    e->last_emit = npad;
    if (cudaMemcpyAsync(next_tokens_out_dev, e->g_next, sizeof(int) * n_active, cudaMemcpyDeviceToDevice, st) !=
        cudaSuccess) {
      cudaError_t ce = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "token copy: %s", cudaGetErrorString(ce));
    }
  }
  if (logits_out_dev) {
    if (cudaMemcpyAsync(logits_out_dev, e->logits, sizeof(float) * (size_t)n_active * e->cfg.n_vocab,
                        cudaMemcpyDeviceToDevice, st) != cudaSuccess) {
      cudaError_t ce = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "logits copy: %s", cudaGetErrorString(ce));
    }
  }
  return WDZ_OK;
}

// ---- decode with the rule state on the device --------------------------------
__global__ void stage_slots_kernel(const int* __restrict__ slots, int n, int npad, int* __restrict__ g_slots) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < npad) g_slots[r] = r < n ? slots[r] : -1;
}

static int ts_step_body(wdz_engine* e, int npad, cudaStream_t st) {
  launch_pdl(e, ts_rules_kernel, dim3((npad + 127) / 128), dim3(128), 0, st, (const int*)e->g_slots, npad,
             (const TsState*)e->ts_state, e->cfg.n_slots, e->ts_params, e->g_rules, e->g_tokens);
  WDZ_LAUNCH_CHECK(e, "ts_rules");
  int rc = decode_step_body(e, e->g_tokens, e->g_slots, e->g_rules, npad, e->g_next, st);
  if (rc) return rc;
  launch_pdl(e, ts_update_kernel, dim3((npad + 127) / 128), dim3(128), 0, st, e->g_slots, npad,
             (const int*)e->g_next, e->ts_state, e->cfg.n_slots, e->ts_params, e->ts_log, e->cfg.max_tokens);
  WDZ_LAUNCH_CHECK(e, "ts_update");
  return WDZ_OK;
}

int wdz_ts_configure(wdz_engine* e, int eot, int ts_begin, int ts_end, int first_timing_max,
                     int open_after_close_span, uint32_t bit_special, uint32_t bit_timings) {
  if (!e) return WDZ_EINVAL;
  if (eot < 0 || ts_begin < 0 || ts_end < ts_begin || ts_end >= e->cfg.n_vocab || eot >= e->cfg.n_vocab)
    return e->fail(WDZ_EINVAL, "wdz_ts_configure: token ids outside the vocabulary");
  e->ts_params = TsParams{eot, ts_begin, ts_end, first_timing_max, open_after_close_span, bit_special, bit_timings};
  for (auto& g : e->ts_graphs) cudaGraphExecDestroy(g.second.exec);   // captured graphs carry the old constants
  e->ts_graphs.clear();
  return WDZ_OK;
}

int wdz_ts_reset(wdz_engine* e, const int32_t* slot_ids_dev, const int32_t* max_new_dev, int n, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!slot_ids_dev || !max_new_dev || n < 0) return e->fail(WDZ_EINVAL, "wdz_ts_reset: null argument");
  if (n == 0) return WDZ_OK;
  ts_reset_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)s>>>(slot_ids_dev, max_new_dev, n, e->ts_state,
                                                                 e->cfg.n_slots);
  WDZ_LAUNCH_CHECK(e, "ts_reset");
  return WDZ_OK;
}

int wdz_ts_first(wdz_engine* e, const float* logits_dev, const int32_t* slot_ids_dev, int n, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!logits_dev || !slot_ids_dev || n < 0) return e->fail(WDZ_EINVAL, "wdz_ts_first: null argument");
  if (n == 0) return WDZ_OK;
  if (n > e->cfg.max_rows) return e->fail(WDZ_ECAPACITY, "wdz_ts_first: %d rows > max_rows %d", n, e->cfg.max_rows);
  cudaStream_t st = (cudaStream_t)s;
  ts_rules_kernel<<<(n + 127) / 128, 128, 0, st>>>(slot_ids_dev, n, e->ts_state, e->cfg.n_slots, e->ts_params,
                                                    e->g_rules, e->g_tokens);
  WDZ_LAUNCH_CHECK(e, "ts_rules");
  if ((rc = rules_launch(e, logits_dev, nullptr, e->g_rules, n, 1, e->g_next, st))) return rc;
  // the update kernel edits its row list in place (finished rows are dropped): work on the staged copy
  stage_slots_kernel<<<(n + 127) / 128, 128, 0, st>>>(slot_ids_dev, n, n, e->g_slots);
  ts_update_kernel<<<(n + 127) / 128, 128, 0, st>>>(e->g_slots, n, e->g_next, e->ts_state, e->cfg.n_slots,
                                                     e->ts_params, e->ts_log, e->cfg.max_tokens);
  WDZ_LAUNCH_CHECK(e, "ts_update");
  return WDZ_OK;
}

int wdz_ts_steps(wdz_engine* e, const int32_t* slot_ids_dev, int n, int k, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!slot_ids_dev || n < 0 || k < 0) return e->fail(WDZ_EINVAL, "wdz_ts_steps: bad argument");
  if (n == 0 || k == 0) return WDZ_OK;
  const int cap = e->cfg.max_rows < e->max_emit ? e->cfg.max_rows : e->max_emit;
  if (n > cap) return e->fail(WDZ_ECAPACITY, "wdz_ts_steps: %d rows > capacity %d", n, cap);
  cudaStream_t st = (cudaStream_t)s;
  int npad = (n + 7) / 8 * 8;
  if (npad > cap) npad = n;
  stage_slots_kernel<<<(npad + 127) / 128, 128, 0, st>>>(slot_ids_dev, n, npad, e->g_slots);
  WDZ_LAUNCH_CHECK(e, "stage_slots");
  const bool use_graph = !(e->cfg.flags & WDZ_FLAG_NO_GRAPH) && !e->profiling;
  if (!use_graph) {
    for (int i = 0; i < k; ++i)
      if ((rc = ts_step_body(e, npad, st))) return rc;
    e->last_emit = npad;
    return WDZ_OK;
  }
  auto it = e->ts_graphs.find(npad);
  if (it == e->ts_graphs.end()) {
    const long long before = e->launches;
    cudaGraph_t graph = nullptr;
    if (!e->cap_stream && cudaStreamCreateWithFlags(&e->cap_stream, cudaStreamNonBlocking) != cudaSuccess) {
      cudaError_t ce0 = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "capture stream: %s", cudaGetErrorString(ce0));
    }
    if (cudaStreamBeginCapture(e->cap_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaError_t ce0 = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "graph capture begin: %s", cudaGetErrorString(ce0));
    }
    rc = ts_step_body(e, npad, e->cap_stream);
    cudaError_t ce = cudaStreamEndCapture(e->cap_stream, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (ce != cudaSuccess || !graph) {
      cudaGetLastError();
      return e->fail(WDZ_ECUDA, "graph capture end: %s", cudaGetErrorString(ce));
    }
    wdz_engine::StepGraph g{};
    ce = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) {
      cudaGetLastError();
      return e->fail(WDZ_ECUDA, "graph instantiate: %s", cudaGetErrorString(ce));
    }
    g.launches = e->launches - before;
    e->launches = before;
    it = e->ts_graphs.emplace(npad, g).first;
  }
  for (int i = 0; i < k; ++i) {
    if (cudaGraphLaunch(it->second.exec, st) != cudaSuccess) {
      cudaError_t ce = cudaGetLastError();
      return e->fail(WDZ_ECUDA, "graph launch: %s", cudaGetErrorString(ce));
    }
    e->launches += it->second.launches;
  }
  e->last_emit = npad;
  return WDZ_OK;
}

int wdz_ts_poll(wdz_engine* e, int32_t* out_host, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!out_host) return e->fail(WDZ_EINVAL, "wdz_ts_poll: null argument");
  cudaStream_t st = (cudaStream_t)s;
  // the status word rides along with the state download: an exhausted wait or a NaN row in any kernel since the
  // last poll turns this call into an error without a synchronisation of its own
  DevStatus h{};
  if (cudaMemcpyAsync(out_host, e->ts_state, sizeof(TsState) * e->cfg.n_slots, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaMemcpyAsync(&h, e->status, sizeof h, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "rule state read: %s", cudaGetErrorString(ce));
  }
  if (h.code != 0) {
    cudaMemsetAsync(e->status, 0, sizeof(DevStatus), st);
    return e->fail(h.code, "device reported status %d (detail %d)", h.code, h.detail);
  }
  return WDZ_OK;
}

int wdz_ts_tokens(wdz_engine* e, int slot, int32_t* out_host, int cap, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!out_host || slot < 0 || slot >= e->cfg.n_slots || cap < 0) return e->fail(WDZ_EINVAL, "wdz_ts_tokens: bad argument");
  if (cap > e->cfg.max_tokens) cap = e->cfg.max_tokens;
  cudaStream_t st = (cudaStream_t)s;
  if (cudaMemcpyAsync(out_host, e->ts_log + (size_t)slot * e->cfg.max_tokens, sizeof(int) * cap,
                      cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
    cudaError_t ce = cudaGetLastError();
    return e->fail(WDZ_ECUDA, "token log read: %s", cudaGetErrorString(ce));
  }
  return WDZ_OK;
}

int wdz_reargmax(wdz_engine* e, const int32_t* rows_dev, const wdz_rule_desc* rules_dev, int n, int32_t* out_dev,
                 wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!rows_dev || !out_dev || n < 0) return e->fail(WDZ_EINVAL, "wdz_reargmax: null argument");
  if (n > e->last_emit) return e->fail(WDZ_EINVAL, "wdz_reargmax: %d rows but only %d logit rows are held", n, e->last_emit);
  return rules_launch(e, e->logits, rows_dev, rules_dev, n, 0, out_dev, (cudaStream_t)s);
}

int wdz_rules_argmax(wdz_engine* e, const float* logits_dev, const wdz_rule_desc* rules_dev, int n,
                     int apply_penalty, int32_t* out_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!logits_dev || !out_dev || n < 0) return e->fail(WDZ_EINVAL, "wdz_rules_argmax: null argument");
  return rules_launch(e, logits_dev, nullptr, rules_dev, n, apply_penalty ? 1 : 0, out_dev, (cudaStream_t)s);
}

// ---- word-timing alignment -------------------------------------------------
}  // extern "C"

#ifdef WDZ_WITH_TC
// Teacher-forced pass over whole chunks (bf16): n = n_chunks * t_pad rows, chunk-major.  The rows of a chunk only
// attend to each other (causally) and to the chunk's cross cache, so nothing is appended to the self cache:
// Q, K and V of a layer are the columns of one bf16 [n, 3d] product, exactly the encoder's layout, and every
// product runs on the 128 x 256 tcgen05 GEMM with its weights read once for all rows.
static int align_pass_tc(wdz_engine* e, const int* tokens, int n, int n_chunks, int t_pad, const int* chunk_lens,
                         const int* chunk_slots, const AlignCapture& cap, cudaStream_t s) {
  const wdz_config& c = e->cfg;
  const int d = c.n_text_state, H = c.n_text_head;
  int rc;
  bf16* xn = (bf16*)e->dxn;
  bf16* ao = (bf16*)e->dao;
  bf16* hid = (bf16*)e->dh;
  bf16* qkvb = (bf16*)e->dqkv;
  bf16* qb = (bf16*)e->dq;
  embed_kernel<bf16><<<n, 256, 0, s>>>(tokens, e->al_pos, (const bf16*)e->tok_emb, (const bf16*)e->dec_pos, e->dx, n, d, c.n_vocab,
                                       c.n_text_ctx);
  e->launches += 1;
  WDZ_LAUNCH_CHECK(e, "embed");
  for (int l = 0; l <= e->al_last_layer && l < c.n_text_layer; ++l) {
    const LayerW& w = e->dec[l];
    if ((rc = launch_ln<bf16, bf16>(e, e->dx, d, nullptr, w.ln1_w, w.ln1_b, xn, d, n, d, s))) return rc;
    if ((rc = enc_gemm<bf16>(e, EPI_STORE, dense_params(xn, d, w.qkv_w, w.qkv_b, qkvb, 3 * d, n, 3 * d, d), s))) return rc;
    if ((rc = attn_tc_launch(e, qkvb, ao, n_chunks, t_pad, d, H, s, chunk_lens, true))) return rc < 0 ? rc : e->fail(WDZ_EINVAL, "alignment: attention shape");
    if ((rc = enc_gemm<bf16>(e, EPI_RESID, dense_params(ao, d, w.out_w, w.out_b, e->dx, d, n, d, d), s))) return rc;

    if ((rc = launch_ln<bf16, bf16>(e, e->dx, d, nullptr, w.lnx_w, w.lnx_b, xn, d, n, d, s))) return rc;
    if ((rc = enc_gemm<bf16>(e, EPI_STORE, dense_params(xn, d, w.xq_w, w.xq_b, qb, d, n, d, d), s))) return rc;
    int here = 0;
    for (int j = 0; j < e->al_heads.n; ++j) here += e->al_heads.layer[j] == l;
    if (here > 0) {
      align_capture_kernel<bf16><<<n, 64 * here, 0, s>>>(qb, d, n, l, e->al_heads, cap.qcap, cap.rows_total, cap.row_base);
      e->launches += 1;
      WDZ_LAUNCH_CHECK(e, "align_capture");
    }
    if (l >= e->al_last_layer) break;
    if ((rc = attn_tc_chunks_launch(e, qb, ao, e->cross_k, e->cross_v, c.n_audio_ctx, c.n_audio_ctx, l, chunk_lens,
                                    chunk_slots, n_chunks, t_pad, false, s)))
      return rc < 0 ? rc : e->fail(WDZ_EINVAL, "alignment: attention shape");
    if ((rc = enc_gemm<bf16>(e, EPI_RESID, dense_params(ao, d, w.xout_w, w.xout_b, e->dx, d, n, d, d), s))) return rc;

    if ((rc = launch_ln<bf16, bf16>(e, e->dx, d, nullptr, w.ln2_w, w.ln2_b, xn, d, n, d, s))) return rc;
    if ((rc = enc_gemm<bf16>(e, EPI_GELU, dense_params(xn, d, w.fc1_w, w.fc1_b, hid, 4 * d, n, 4 * d, d), s))) return rc;
    if ((rc = enc_gemm<bf16>(e, EPI_RESID, dense_params(hid, 4 * d, w.fc2_w, w.fc2_b, e->dx, d, n, d, 4 * d), s))) return rc;
  }
  return WDZ_OK;
}
#endif

extern "C" {
int wdz_align_configure(wdz_engine* e, const int32_t* layer_head_pairs, int n_heads) {
  if (!e) return WDZ_EINVAL;
  if (!layer_head_pairs || n_heads < 1 || n_heads > ALIGN_MAX_HEADS)
    return e->fail(WDZ_EINVAL, "wdz_align_configure: 1..%d (layer, head) pairs", ALIGN_MAX_HEADS);
  if (e->cfg.n_text_state / e->cfg.n_text_head != ALIGN_HD)
    return e->fail(WDZ_EINVAL, "wdz_align_configure: head size %d is not supported", e->cfg.n_text_state / e->cfg.n_text_head);
  AlignHeads h{};
  int last = -1;
  for (int j = 0; j < n_heads; ++j) {
    const int l = layer_head_pairs[2 * j], hd = layer_head_pairs[2 * j + 1];
    if (l < 0 || l >= e->cfg.n_text_layer || hd < 0 || hd >= e->cfg.n_text_head)
      return e->fail(WDZ_EINVAL, "wdz_align_configure: pair %d = (%d, %d) is outside the decoder", j, l, hd);
    h.layer[j] = l; h.head[j] = hd;
    if (l > last) last = l;
  }
  h.n = n_heads;
  e->al_heads = h;
  e->al_last_layer = last;
  return WDZ_OK;
}

// Scratch of the alignment lives in encoder activations that are idle between encoder calls: queries and column
// statistics in the QKV buffer (this bounds the chunks of one call), the scores [chunks, heads, t_pad, Ta] f32 in
// the MLP hidden buffer, filled and consumed a few chunks at a time.
static int64_t align_score_chunks(const wdz_engine* e, int t_pad) {   // chunks whose scores fit at once
  const wdz_config& c = e->cfg;
  const int64_t hid_bytes = (int64_t)e->esz * c.max_clips * c.n_audio_ctx * 4 * c.n_audio_state;
  return hid_bytes / ((int64_t)e->al_heads.n * t_pad * c.n_audio_ctx * 4);
}
static int64_t align_capacity(const wdz_engine* e, int t_pad) {
  const wdz_config& c = e->cfg;
  if (e->al_heads.n < 1 || t_pad < 1 || align_score_chunks(e, t_pad) < 1) return 0;
  const int64_t qkv_bytes = (int64_t)e->esz * c.max_clips * c.n_audio_ctx * 3 * c.n_audio_state;
  const int64_t per_q = (int64_t)e->al_heads.n * t_pad * ALIGN_HD * 4 + (int64_t)e->al_heads.n * c.n_audio_ctx * 8 + 512;
  return qkv_bytes / per_q;
}

int wdz_align_capacity(wdz_engine* e, int t_pad) {
  if (!e) return WDZ_EINVAL;
  const int64_t n = align_capacity(e, t_pad);
  return n > (1 << 20) ? (1 << 20) : (int)n;
}

int wdz_align_matrix(wdz_engine* e, const int32_t* tokens_dev, const int32_t* chunk_lens_dev,
                     const int32_t* chunk_slots_dev, const int32_t* audio_caps_dev, int n_chunks, int t_pad,
                     float* matrix_out_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  const wdz_config& c = e->cfg;
  if (!tokens_dev || !chunk_lens_dev || !chunk_slots_dev || !audio_caps_dev || !matrix_out_dev || n_chunks < 0)
    return e->fail(WDZ_EINVAL, "wdz_align_matrix: null argument");
  if (e->al_heads.n < 1) return e->fail(WDZ_ESTATE, "wdz_align_matrix: wdz_align_configure has not been called");
  if (n_chunks == 0) return WDZ_OK;
  if (t_pad < 1 || t_pad > c.max_tokens || t_pad > c.n_text_ctx)
    return e->fail(WDZ_ECAPACITY, "wdz_align_matrix: %d tokens per chunk > %d", t_pad, c.max_tokens < c.n_text_ctx ? c.max_tokens : c.n_text_ctx);
  if (c.n_audio_ctx > 32 * ALIGN_COLS_PER_LANE)
    return e->fail(WDZ_ECAPACITY, "wdz_align_matrix: %d audio positions > %d", c.n_audio_ctx, 32 * ALIGN_COLS_PER_LANE);
  if (n_chunks > align_capacity(e, t_pad))
    return e->fail(WDZ_ECAPACITY, "wdz_align_matrix: %d chunks of %d tokens > %lld per call (wdz_align_capacity)", n_chunks,
                   t_pad, (long long)align_capacity(e, t_pad));
  cudaStream_t st = (cudaStream_t)s;
  const int64_t rows = (int64_t)n_chunks * t_pad;
  const int nh = e->al_heads.n, Ta = c.n_audio_ctx;
  float* w = (float*)e->hid;
  float* qcap = (float*)e->qkv;
  float* mean = qcap + (int64_t)nh * rows * ALIGN_HD;
  float* rstd = mean + (int64_t)n_chunks * nh * Ta;
  // bf16 with room for whole chunks in one forward call: attention of the pass on the tensor cores
  bool tc_pass = false;
#ifdef WDZ_WITH_TC
  tc_pass = c.dtype == WDZ_BF16 && !(c.flags & WDZ_FLAG_NO_TENSOR_CORE) && t_pad <= c.max_rows && c.n_text_state % 256 == 0;
#endif
  // the row-wise pass appends to the self-attention rows of the chunks' slots from position 0
  if (!tc_pass) reset_seqlens_kernel<<<(n_chunks + 255) / 256, 256, 0, st>>>(chunk_slots_dev, e->seq_lens, n_chunks, c.n_slots);
  // rows per forward call: whole chunks, and for the tensor-core pass no more 128-row tiles than make the
  // d-wide products (d / 256 column tiles each) one full wave of the SMs; 3d- and 4d-wide ones then take 3 and 4
  int64_t group = c.max_rows;
  if (tc_pass) {
    const int64_t wave_rows = (int64_t)std::max(1, e->sm_count / std::max(1, c.n_text_state / 256)) * 128;
    int64_t cap_rows = std::min<int64_t>(c.max_rows, wave_rows);
    if (cap_rows < t_pad) cap_rows = t_pad;
    group = cap_rows / t_pad * t_pad;
  }
  for (int64_t r0 = 0; r0 < rows; r0 += group) {
    const int n = (int)(rows - r0 < group ? rows - r0 : group);
    align_rows_kernel<<<(n + 255) / 256, 256, 0, st>>>(chunk_slots_dev, chunk_lens_dev, t_pad, (int)r0, n, c.n_slots, e->al_slots, e->al_pos);
    e->launches += 1;
    AlignCapture cap{qcap, rows, r0};
#ifdef WDZ_WITH_TC
    if (tc_pass) {
      rc = align_pass_tc(e, tokens_dev + r0, n, n / t_pad, t_pad, chunk_lens_dev + r0 / t_pad, chunk_slots_dev + r0 / t_pad, cap, st);
      if (rc) return rc;
      continue;
    }
#endif
    rc = c.dtype == WDZ_BF16
             ? forward_rows_impl<bf16>(e, tokens_dev + r0, e->al_slots, e->al_pos, n, nullptr, 0, st, &cap)
             : forward_rows_impl<float>(e, tokens_dev + r0, e->al_slots, e->al_pos, n, nullptr, 0, st, &cap);
    if (rc) return rc;
  }
  const int per = (int)std::min<int64_t>(align_score_chunks(e, t_pad), n_chunks);
  for (int c0 = 0; c0 < n_chunks; c0 += per) {
    const int nb = std::min(per, n_chunks - c0);
    const dim3 gs((t_pad + 7) / 8, nh, nb);
    const int* lens_b = chunk_lens_dev + c0;
    if (c.dtype == WDZ_BF16)
      align_scores_kernel<bf16><<<gs, 256, 0, st>>>(qcap, rows, c0, t_pad, lens_b, chunk_slots_dev + c0, audio_caps_dev + c0,
                                                    e->al_heads, (const bf16*)e->cross_k, c.n_slots, Ta, c.n_text_state, w);
    else
      align_scores_kernel<float><<<gs, 256, 0, st>>>(qcap, rows, c0, t_pad, lens_b, chunk_slots_dev + c0, audio_caps_dev + c0,
                                                     e->al_heads, (const float*)e->cross_k, c.n_slots, Ta, c.n_text_state, w);
    align_colstats_kernel<<<dim3((Ta + 127) / 128, nh, nb), 128, 0, st>>>(w, nh, t_pad, Ta, lens_b, mean, rstd);
    align_matrix_kernel<<<dim3(t_pad, nb), 256, 0, st>>>(w, mean, rstd, nh, t_pad, Ta, lens_b,
                                                         matrix_out_dev + (int64_t)c0 * t_pad * Ta);
    e->launches += 3;
  }
  WDZ_LAUNCH_CHECK(e, "align_matrix");
  return WDZ_OK;
}

int wdz_dtw(wdz_engine* e, const float* matrix_dev, int64_t chunk_stride, int64_t ld, const int32_t* row0_dev,
            const int32_t* n_rows_dev, const int32_t* n_cols_dev, const int32_t* col_lo_dev, const int32_t* col_hi_dev,
            int limit_stride, int n_chunks, int max_rows, int max_cols, int32_t* text_idx_out_dev,
            int32_t* time_idx_out_dev, int32_t* path_len_out_dev, wdz_stream s) {
  int rc = check_ready(e);
  if (rc) return rc;
  if (!matrix_dev || !row0_dev || !n_rows_dev || !n_cols_dev || !text_idx_out_dev || !time_idx_out_dev ||
      !path_len_out_dev || n_chunks < 0 || (!col_lo_dev) != (!col_hi_dev))
    return e->fail(WDZ_EINVAL, "wdz_dtw: null argument");
  if (n_chunks == 0) return WDZ_OK;
  if (max_rows < 1 || max_cols < 1 || max_rows > 511 || dtw_smem_bytes(max_rows, max_cols) > (size_t)200 * 1024)
    return e->fail(WDZ_ECAPACITY, "wdz_dtw: %d x %d cells do not fit one CTA's shared memory (rows <= 511, rows x cols / 4 <= ~200 KB)",
                   max_rows, max_cols);
  if (col_lo_dev && limit_stride < max_rows) return e->fail(WDZ_EINVAL, "wdz_dtw: limit_stride %d < max_rows %d", limit_stride, max_rows);
  if (ld < max_cols || (n_chunks > 1 && chunk_stride < ld)) return e->fail(WDZ_EINVAL, "wdz_dtw: ld %lld < max_cols %d or chunk stride too small", (long long)ld, max_cols);
  DtwParams p{};
  p.mat = matrix_dev; p.chunk_stride = chunk_stride; p.ld = ld;
  p.row0 = row0_dev; p.n_rows = n_rows_dev; p.n_cols = n_cols_dev;
  p.col_lo = col_lo_dev; p.col_hi = col_hi_dev; p.limit_stride = limit_stride;
  p.max_rows = max_rows; p.max_cols = max_cols; p.path_cap = max_rows + max_cols;
  p.text_idx = text_idx_out_dev; p.time_idx = time_idx_out_dev; p.path_len = path_len_out_dev;
  p.status = e->status;
  dtw_kernel<<<n_chunks, 512, dtw_smem_bytes(max_rows, max_cols), (cudaStream_t)s>>>(p);
  e->launches += 1;
  WDZ_LAUNCH_CHECK(e, "dtw");
  return WDZ_OK;
}

}  // extern "C"
