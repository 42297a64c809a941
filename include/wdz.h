/*
 * wdz.h - C ABI of the B200 transcription engine (libwdz.so).
 *
 * The reference project is pure Python and has no FFI of its own; its seam is
 * the set of methods its Transcriber calls on the model object.  Each entry
 * point below names the reference call it stands in for (paths inside the
 * reference project).  Conventions:
 *   - every function returns WDZ_OK (0) or a negative WDZ_E* code and never
 *     throws or aborts; wdz_last_error() gives the text of the last failure;
 *   - all buffers are caller-owned device memory (the Python host passes
 *     torch ``data_ptr()`` values); "dev" in a comment means a device pointer,
 *     "host" a host pointer; the engine allocates nothing on the device;
 *   - calls are asynchronous on the given stream unless they fill host memory;
 *   - an engine is not thread-safe; use one engine per GPU per process.
 */
#ifndef WDZ_H_
#define WDZ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WDZ_OK 0
#define WDZ_EINVAL (-1)    /* bad argument */
#define WDZ_ENOMEM (-2)    /* workspace missing or too small */
#define WDZ_ECUDA (-3)     /* a CUDA call failed */
#define WDZ_ESTATE (-4)    /* engine not finalized, or a tensor was never bound */
#define WDZ_ECAPACITY (-5) /* more clips / rows / slots than the engine was built for */
#define WDZ_ENAN (-6)      /* a row of logits held NaN */
#define WDZ_ETIMEOUT (-7)  /* a bounded device-side wait ran out */

#define WDZ_F32 0
#define WDZ_BF16 1

typedef void* wdz_stream; /* a cudaStream_t */
typedef struct wdz_engine wdz_engine;

/* Shape of the model plus the capacities the workspace is sized for.  The
 * first ten fields are the reference's ModelDimensions
 * (src/whisperdrz/config.py:4-15). */
typedef struct wdz_config {
  int32_t n_mels, n_audio_ctx, n_audio_state, n_audio_head, n_audio_layer;
  int32_t n_vocab, n_text_ctx, n_text_state, n_text_head, n_text_layer;
  int32_t dtype;      /* WDZ_F32 or WDZ_BF16: type of weights, KV caches, encoder output */
  int32_t n_slots;    /* KV slots (reference: BS + n_warm, transcriber.py:566-568) */
  int32_t max_tokens; /* self-attention cache length per slot (transcriber.py:673-677) */
  int32_t max_clips;  /* most 30 s windows per wdz_logmel / wdz_encode / wdz_cross_kv call */
  int32_t max_rows;   /* most token rows per wdz_forward_rows / wdz_decode_step call */
  int32_t flags;      /* WDZ_FLAG_* */
} wdz_config;

#define WDZ_FLAG_NO_TENSOR_CORE 1 /* keep bf16 GEMMs on the CUDA-core path (debug / A-B runs) */
#define WDZ_FLAG_NO_GRAPH 4       /* launch the decode step kernel by kernel instead of replaying a CUDA graph */
#define WDZ_FLAG_NO_PDL 8         /* decode kernels launched without programmatic dependent launch */
#define WDZ_FLAG_NO_SPLIT_STEP 32 /* decode steps of many rows as one batch on one stream (no half-batch overlap) */
#define WDZ_FLAG_NO_CTA_PAIRS 16  /* encoder-shaped GEMMs on lone CTAs (128x256 tiles) instead of CTA pairs (256x256) */
#define WDZ_FLAG_NO_BULK_COPY 2   /* cross-attention through plain loads instead of the bulk-copy ring */

/* Per-row logit rule: the device half of decode_batch
 * (src/whisperdrz/decoding.py:1514-1777).  Blocked set of a row =
 *   base(mode) | OR of tables whose bit is set in table_bits | table or_table
 *   | complement of table allow_table
 *   | ids in [prefix_begin, prefix_end) | set_ids[0..n_set)
 * with clear_ids[0..n_clear) removed last.  This is the normal form of the
 * reference's ordered mask steps: its "block everything, then enable a class"
 * overrides become the base mode, its per-language base set is or_table, its
 * tag-prefix allow list (decoding.py:1623-1639) is allow_table, its
 * backwards-timestamp block (:1682-1689) the prefix range.
 * Tables are bitsets over the vocabulary, bound as "rules.tables"
 * ([n_tables][ceil(n_vocab / 32)] uint32, n_tables >= WDZ_MAX_TABLES): the first
 * WDZ_MAX_TABLES can be OR-ed through table_bits, any table can be named by
 * arg0 (WDZ_MODE_ALL_EXCEPT_TABLE), or_table and allow_table; there 0 means
 * "none", so table 0 itself cannot be named by those two fields.
 * Blocked ids get -65504 added (decoding.py:1725-1729); ids in pen_ids get the
 * repetition penalty v > 0 ? v / 1.2 : v * 1.2 (decoding.py:1733-1759); then
 * argmax, lowest id winning ties.  forced_id >= 0 skips all of that and returns
 * forced_id (rows decided on the host, decoding.py:1098-1456). */
#define WDZ_MODE_OR 0               /* base = nothing blocked */
#define WDZ_MODE_ALL_EXCEPT_TABLE 1 /* base = everything blocked except table arg0 */
#define WDZ_MODE_ALL_EXCEPT_RANGE 2 /* base = everything blocked except ids [arg0, arg1) */
#define WDZ_MODE_ALL 3              /* base = everything blocked (use clear_ids) */
#define WDZ_MAX_TABLES 32
typedef struct wdz_rule_desc {
  int32_t forced_id;
  int32_t mode, arg0, arg1;
  uint32_t table_bits;
  int32_t prefix_begin, prefix_end;
  int32_t n_set, set_ids[6];
  int32_t or_table;    /* 0 = none, else index of one more table to OR in */
  int32_t allow_table; /* 0 = none, else index of a table whose complement is blocked */
  int32_t n_clear, clear_ids[4];
  int32_t n_pen, pen_ids[10];
} wdz_rule_desc; /* 32 x int32 = 128 bytes */

/* ---- life cycle ------------------------------------------------------- */
/* Stands in for WhisperDRZ.__init__ + Transcriber.load_model
 * (model.py:649-693, transcriber.py:642-726). */
int wdz_engine_create(const wdz_config* cfg, wdz_engine** out);
int wdz_engine_destroy(wdz_engine* e);
/* Scratch the engine needs for the capacities in its config. */
int wdz_workspace_bytes(const wdz_engine* e, size_t* out_bytes);
int wdz_set_workspace(wdz_engine* e, void* dev, size_t bytes);
/* Lend the engine one tensor (dtype = cfg.dtype unless noted).  Names are
 * those produced by pack_weights in whisperdrz_b200/engine.py: the reference's
 * state_dict tensors (model.py:258-261,387-394,449-461,493-529), with q/k/v
 * stacked per attention and the conv kernels tap-major, plus
 *   cache.self_k / cache.self_v   [n_text_layer, n_slots, max_tokens, n_text_state]
 *   cache.cross_k / cache.cross_v [n_text_layer, n_slots, n_audio_ctx, n_text_state]
 *   cache.seq_lens                int32 [n_slots]
 * (FlashKVCache, model.py:98-147, one allocation per kind instead of one
 * object per layer) and rules.tables uint32 [n_tables >= WDZ_MAX_TABLES, ceil(n_vocab/32)]
 * (the [V] bool class masks of DecoderState, decoding.py:397-724, as bitsets; optional). */
int wdz_bind(wdz_engine* e, const char* name, const void* dev, int64_t numel);
int wdz_finalize(wdz_engine* e);
const char* wdz_last_error(const wdz_engine* e);
const char* wdz_version(void);
/* Reads and clears the device-side error word (WDZ_OK, WDZ_ENAN, WDZ_ETIMEOUT).
 * Synchronises the stream. */
int wdz_device_status(wdz_engine* e, wdz_stream s);

/* ---- measurement (no counterpart in the reference, which ships no profiling) ---- */
#define WDZ_PROF_CROSS_ATTN 0 /* decode cross-attention kernel; work = K/V bytes read */
#define WDZ_PROF_SELF_ATTN 1  /* decode self-attention kernel; work not tracked (0) */
#define WDZ_PROF_DEC_GEMM 2   /* decode-shaped products; work = weight bytes */
#define WDZ_PROF_ENC_GEMM 3   /* encoder / conv / cross-KV products; work = flops */
#define WDZ_PROF_ENC_ATTN 4   /* encoder attention; work = flops */
#define WDZ_PROF_LM_HEAD 5    /* tied LM head; work = weight bytes */
#define WDZ_PROF_LOGMEL 6     /* the three log-mel kernels together */
/* Kernels enqueued by this engine since it was created. */
int wdz_launch_count(const wdz_engine* e, int64_t* out);
/* enable != 0: start recording a CUDA-event pair around every launch of the
 * kinds above (and forget earlier records); 0: stop.  Recording costs a few
 * microseconds per launch, so headline timings are taken with it off. */
int wdz_profile(wdz_engine* e, int enable);
/* Synchronises the device, then sums the recorded launches of one kind. */
int wdz_profile_read(wdz_engine* e, int kind, double* total_ms, int64_t* launches, double* work);

/* ---- front end: LogMelSpectrogram.forward (audio.py:108-156) ----------- */
/* audio_dev f32 [B, audio_stride]; n_samples_dev int32 [B] (>= 400 each, the
 * reflect padding needs it); frame_offset_dev int32 [B] or NULL: first frame
 * of the 3000-frame window (continuation windows, transcriber.py:1062-1072).
 * mel_out_dev f32 [B, n_mels, 3000]; frames past the clip are -1.5. */
int wdz_logmel(wdz_engine* e, const float* audio_dev, int64_t audio_stride,
               const int32_t* n_samples_dev, const int32_t* frame_offset_dev, int B,
               float* mel_out_dev, wdz_stream s);

/* wdz_logmel for hosts that cannot hand the engine a workspace.  No counterpart
 * in the reference (its front end runs in torch on the CPU and allocates
 * freely).  Some embedders of this library run inside a process whose GPU
 * memory is handed out in full to another pool at start-up (a serving process
 * that gives everything to its KV-cache manager), or inside a loop where the
 * device-wide stall of cudaMalloc / cudaFree is not acceptable; they can bind
 * the weights and tables they already hold but have nothing left to lend as
 * scratch.  This entry point therefore takes no workspace: the un-normalised
 * log-mel and the per-clip maxima go into an array compiled into the library
 * (WDZ_STATIC_MAX_CLIPS x WDZ_STATIC_MAX_MELS x 3000 floats, about 6.1 MB,
 * resident on every GPU that loads the library until the process exits).  It
 * calls no cudaMalloc, cudaFree or allocating library routine; wdz_set_workspace
 * need not have been called.  Same arguments and results as wdz_logmel, with
 * B <= WDZ_STATIC_MAX_CLIPS and cfg.n_mels <= WDZ_STATIC_MAX_MELS, otherwise
 * WDZ_ECAPACITY.  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress); make that first call before any stream
 * capture begins.  All calls share the one array: it keeps the previous
 * call's contents (the maxima are re-initialised inside every call), and two
 * calls that overlap on the GPU - different streams or engines - race on it. */
#define WDZ_STATIC_MAX_CLIPS 4
#define WDZ_STATIC_MAX_MELS 128
int wdz_logmel_static(wdz_engine* e, const float* audio_dev, int64_t audio_stride,
                      const int32_t* n_samples_dev, const int32_t* frame_offset_dev, int B,
                      float* mel_out_dev, wdz_stream s);

/* ---- encoder: AudioEncoder.forward (model.py:462-475) ------------------ */
/* mel_dev f32 [B, n_mels, 3000] -> xa_out_dev [B, n_audio_ctx, n_audio_state] in cfg.dtype */
int wdz_encode(wdz_engine* e, const float* mel_dev, int B, void* xa_out_dev, wdz_stream s);

/* One nn.Linear (+ exact GELU when gelu != 0) in cfg.dtype, as the encoder
 * runs it (model.py:258-261, 387-393): y[M,N] = act(x[M,K] w[N,K]^T + bias).
 * bias_dev may be NULL.  cuda_cores_only (for A/B checks): 1 keeps a bf16
 * product off the tcgen05 kernels, 2 keeps it on the lone-CTA tcgen05 kernel
 * (no CTA pairs), 0 is the engine's own choice. */
int wdz_linear(wdz_engine* e, const void* x_dev, int M, int K, const void* w_dev, const void* bias_dev, int N,
               int gelu, void* y_dev, int cuda_cores_only, wdz_stream s);

/* One nn.Linear as the decoder runs it for a handful of token rows
 * (model.py:258-261 called from forward_flash): x_dev [M, K] in cfg.dtype,
 * w_dev [N, K], optional bias -> y_dev f32 [M, N]; accumulate != 0 adds into
 * y_dev (the residual-stream update of model.py:421-434) instead of storing. */
int wdz_linear_rows(wdz_engine* e, const void* x_dev, int M, int K, const void* w_dev, const void* bias_dev, int N,
                    int accumulate, float* y_dev, wdz_stream s);

/* Encoder self-attention alone (MultiHeadAttention.qkv_attention, model.py:276-298):
 * qkv_dev [B, n_audio_ctx, 3 * n_audio_state] (q | k | v per row, cfg.dtype) ->
 * out_dev [B, n_audio_ctx, n_audio_state]; non-causal, scale 1/8.
 * cuda_cores_only != 0 keeps a bf16 call off the tcgen05 kernel. */
int wdz_encoder_attention(wdz_engine* e, const void* qkv_dev, int B, void* out_dev, int cuda_cores_only,
                          wdz_stream s);

/* ---- decoder ----------------------------------------------------------- */
/* Cross K/V of all layers for B windows into their slots
 * (WhisperDRZ.prefill_flash, model.py:852-855). slot_ids_dev int32 [B]. */
int wdz_cross_kv(wdz_engine* e, const void* xa_dev, const int32_t* slot_ids_dev, int B,
                 wdz_stream s);
/* seq_lens[slot] = 0 (reset_flash_kv, model.py:813-822; prefill_flash :858-862). */
int wdz_slot_reset(wdz_engine* e, const int32_t* slot_ids_dev, int n, wdz_stream s);
/* Copies cache.seq_lens to host (FlashKVCache.seq_lens, read at transcriber.py:1676). Synchronises. */
int wdz_slot_seqlens(wdz_engine* e, int32_t* out_host, wdz_stream s);

/* TextDecoder.forward_flash (model.py:570-617) over ragged rows: row i feeds
 * token tokens_dev[i] at position positions_dev[i] of slot slot_ids_dev[i];
 * its K/V are appended there and it attends causally to [0, position] of that
 * slot and to all encoder positions.  Rows of one slot must carry distinct
 * positions (a prompt is P rows with positions 0..P-1).  Afterwards
 * seq_lens[slot] = max(seq_lens[slot], position + 1).  Logits (f32 [n_emit,
 * n_vocab]) are produced for rows emit_rows_dev[0..n_emit) only (NULL = all n
 * rows); logits_out_dev may be NULL to keep them only inside the engine. */
int wdz_forward_rows(wdz_engine* e, const int32_t* tokens_dev, const int32_t* slot_ids_dev,
                     const int32_t* positions_dev, int n, const int32_t* emit_rows_dev, int n_emit,
                     float* logits_out_dev, wdz_stream s);
/* prefill_flash (model.py:824-869): cross K/V + slot reset for the B windows,
 * then wdz_forward_rows over the flattened prompt rows. */
int wdz_prefill(wdz_engine* e, const void* xa_dev, const int32_t* window_slot_ids_dev, int B,
                const int32_t* tokens_dev, const int32_t* slot_ids_dev, const int32_t* positions_dev,
                int n, const int32_t* emit_rows_dev, int n_emit, float* logits_out_dev, wdz_stream s);
/* One decode step for n_active rows (the loop body of transcriber.py:1666-1702):
 * positions are read from cache.seq_lens on the device, logits stay resident
 * in the engine, rules (NULL = plain argmax) are applied and the chosen ids
 * written to next_tokens_out_dev int32 [n_active] (-1 for a NaN row).
 * logits_out_dev: optional f32 [n_active, n_vocab] copy. */
int wdz_decode_step(wdz_engine* e, const int32_t* tokens_dev, const int32_t* slot_ids_dev, int n_active,
                    const wdz_rule_desc* rules_dev, int32_t* next_tokens_out_dev,
                    float* logits_out_dev, wdz_stream s);
/* ---- decode with the token-level rule state on the device --------------------
 * The timestamp-pair rules (timestamps in open/close pairs, never backwards,
 * first one early, specials never sampled, EOT only between pairs, repetition
 * penalty on the last ten text tokens, forced EOT at the budget: the part of
 * decode_batch / update_state_after_decode, decoding.py:878-963 and 1098-1777,
 * that needs no text) depend on a few integers per slot.  Kept on the device
 * they remove the reference's per-step host round trip: k decode steps are
 * queued by one call and the host only polls.  Class table 0 must hold the
 * special tokens and table 1 the timestamp tokens (or pass other bits to
 * wdz_ts_configure; defaults are the multilingual ids 50257 / 50365..51865). */
int wdz_ts_configure(wdz_engine* e, int eot, int ts_begin, int ts_end, int first_timing_max,
                     int open_after_close_span, uint32_t bit_special, uint32_t bit_timings);
/* Fresh state for the given slots; max_new_dev int32 [n] = token budget of each (EOT is forced at it). */
int wdz_ts_reset(wdz_engine* e, const int32_t* slot_ids_dev, const int32_t* max_new_dev, int n, wdz_stream s);
/* First token after a prefill: logits_dev f32 [n, n_vocab] of the last prompt position of each slot. */
int wdz_ts_first(wdz_engine* e, const float* logits_dev, const int32_t* slot_ids_dev, int n, wdz_stream s);
/* k decode steps for the n slots: each step feeds every slot its last token, applies its rule, argmax,
 * updates its state and appends the token to its log.  Finished slots keep producing EOT until dropped. */
int wdz_ts_steps(wdz_engine* e, const int32_t* slot_ids_dev, int n, int k, wdz_stream s);
/* Copies all slot states to host (24 x int32 per slot: max_new, n_new, timing_count, last_timing,
 * last_was_timing, n_recent, done, last_token, recent[10], 6 spare).  Synchronises the stream.
 * The device status word is read in the same round trip: when a kernel since the last poll gave up a
 * bounded wait or met a NaN logits row, the call returns that code (WDZ_ETIMEOUT, WDZ_ENAN) and clears it. */
int wdz_ts_poll(wdz_engine* e, int32_t* out_host, wdz_stream s);
/* Copies the first cap generated tokens of one slot to host.  Synchronises the stream. */
int wdz_ts_tokens(wdz_engine* e, int slot, int32_t* out_host, int cap, wdz_stream s);

/* Phase-4 re-argmax (decoding.py:2033-2044, _sample_masked :2049-2067) on the
 * logits of the last wdz_decode_step / wdz_forward_rows: rows_dev[i] indexes
 * that call's logit rows; no repetition penalty. */
int wdz_reargmax(wdz_engine* e, const int32_t* rows_dev, const wdz_rule_desc* rules_dev, int n,
                 int32_t* out_dev, wdz_stream s);
/* Phase 3 on caller-held logits f32 [n, n_vocab] (e.g. the first token after
 * a prefill, transcriber.py:1109-1126). */
int wdz_rules_argmax(wdz_engine* e, const float* logits_dev, const wdz_rule_desc* rules_dev, int n,
                     int apply_penalty, int32_t* out_dev, wdz_stream s);

/* ---- word-timing alignment (the step after decode of every finished window) ----
 * Device steps of fill_word_timings_batch (src/whisperdrz/dtw_align.py:1112-1240); text parsing and
 * re-rendering stay host code on the caller's side.
 *
 * wdz_align_configure: the (layer, head) pairs whose cross-attention tracks time; replaces the head mask
 * of make_head_mask (dtw_align.py:52-62).  layer_head_pairs is host int32 [n_heads][2], n_heads <= 16. */
int wdz_align_configure(wdz_engine* e, const int32_t* layer_head_pairs, int n_heads);
/* Most chunks of t_pad tokens one wdz_align_matrix call takes (its scratch is the idle encoder workspace). */
int wdz_align_capacity(wdz_engine* e, int t_pad);
/* Replaces model.decoder(full_tokens, xa_batch) under CrossAttnCapture, compute_attention and
 * _dtw_prep_batch (dtw_align.py:1181-1195, 498-586, 700-753).  Chunk b holds chunk_lens_dev[b] tokens
 * (sot sequence, no-timestamps, ids, eot) at tokens_dev[b * t_pad ...], eot-padded, and is aligned against
 * the audio window whose cross keys sit in slot chunk_slots_dev[b] (written by wdz_cross_kv / wdz_prefill).
 * Runs the decoder teacher-forced up to the last configured layer, takes QK^T of the configured heads
 * against the cached cross keys, softmax over the audio columns below audio_caps_dev[b], normalises each
 * (head, column) over the chunk's rows, median-filters (width 7, reflect) along audio and averages the
 * heads.  matrix_out_dev: f32 [n_chunks][t_pad][n_audio_ctx], rows past a chunk's length zero.
 * bf16 engines with max_rows >= t_pad run the pass for whole chunks on the tensor cores and leave the self
 * cache alone.  Otherwise the pass goes row by row through the decode kernels: it then writes the
 * self-attention rows of the chunks' slots from position 0 (their decoded window is finished), resets those
 * slots' lengths, and the slots of one call must be distinct. */
int wdz_align_matrix(wdz_engine* e, const int32_t* tokens_dev, const int32_t* chunk_lens_dev,
                     const int32_t* chunk_slots_dev, const int32_t* audio_caps_dev, int n_chunks, int t_pad,
                     float* matrix_out_dev, wdz_stream s);
/* Replaces _dtw_numba on the negated matrix with the anchor bands of _apply_anchor_bands
 * (dtw_align.py:170-223, 589-641).  Chunk b's cost is -matrix[b * chunk_stride + (row0[b] + i) * ld + j]
 * for i < n_rows[b], j < n_cols[b], and +inf where j is outside [col_lo[b][i], col_hi[b][i])
 * (int32 [n_chunks][limit_stride]; both NULL = no limits).  Outputs the monotonic minimum-cost path from
 * (0, 0) to the last cell: text_idx / time_idx int32 [n_chunks][max_rows + max_cols] in forward order and
 * its length.  max_rows <= 511 and max_rows * max_cols / 4 within one CTA's shared memory (~200 KB). */
int wdz_dtw(wdz_engine* e, const float* matrix_dev, int64_t chunk_stride, int64_t ld, const int32_t* row0_dev,
            const int32_t* n_rows_dev, const int32_t* n_cols_dev, const int32_t* col_lo_dev, const int32_t* col_hi_dev,
            int limit_stride, int n_chunks, int max_rows, int max_cols, int32_t* text_idx_out_dev,
            int32_t* time_idx_out_dev, int32_t* path_len_out_dev, wdz_stream s);

#ifdef __cplusplus
}
#endif
#endif /* WDZ_H_ */
