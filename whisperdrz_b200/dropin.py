"""Hand-over of the reference ``Transcriber`` to the CUDA engine.

``whisperdrz.Transcriber(model_path=None, model=B200Model(...))`` already runs
on the engine through the model seam (encoder, prefill, decode step).  ``bind``
finishes the job for the three places where the reference scheduler reaches
past that seam (src/whisperdrz/transcriber.py):

* the log-mel front end, which it runs on the CPU (``self.tomel``, :667-668,
  919-925, 1092) -> the engine's fused log-mel kernels;
* its bucketed CUDA graphs of ``forward_flash`` (:31-173, 717-726), whose padded
  rows re-run stale slots -> the engine's own captured step, which pads with
  rows that every kernel skips;
* word timing (``fill_word_timings_batch``, dtw_align.py:1112-1303), which hooks
  ``nn.Module`` projections the engine does not have -> the same host text
  handling (the reference's own functions, called as they are) around the
  engine's teacher-forced pass, cost matrix and DTW (``alignment.align_chunks``).

    import whisperdrz
    from whisperdrz_b200 import dropin
    from whisperdrz_b200.model import B200Model
    t = whisperdrz.Transcriber(model_path=None, model=B200Model(dims, state_dict, tokenizer=tok), lang="en")
    dropin.bind(t)
    t.transcribe(audio)

Everything else - chunking, ``decode_batch`` and its text rules, stop rules,
continuation windows, ``[CHOP]`` stitching, the clean-up chain - is the
reference's own code, untouched.
"""
from __future__ import annotations

import sys
from collections import defaultdict

import torch

from . import alignment
from .model import B200Model


class EngineLogMel:
    """Stands in for ``LogMelSpectrogram`` (audio.py:81-156) as the Transcriber calls it: audio f32 [B, N] on
    the host (or [N]) -> log-mel [B, n_mels, N // 160] (``target_frames`` pads with -1.5 / trims) on the
    engine's device.  Audio the engine's window cannot hold (more than 30 s, or too short to reflect-pad)
    goes to the reference's own module."""

    def __init__(self, model: B200Model, host_module):
        self.model, self.host_module = model, host_module

    def __call__(self, audio: torch.Tensor, target_frames: int | None = None) -> torch.Tensor:
        squeeze = audio.dim() == 1
        a = audio[None] if squeeze else audio
        eng = self.model.engine
        B, N = a.shape
        if eng is None or N > 480000 or N < 400:
            return self.host_module(audio, target_frames=target_frames)
        frames = N // 160
        outs = []
        for i in range(0, B, eng.max_clips):
            blk = a[i: i + eng.max_clips].to(eng.device, torch.float32)
            outs.append(eng.logmel(blk)[:, :, :frames])
        mel = torch.cat(outs, 0)
        if target_frames is not None:
            if frames < target_frames:
                mel = torch.nn.functional.pad(mel, (0, target_frames - frames), value=-1.5)
            mel = mel[:, :, :target_frames]
        return mel[0] if squeeze else mel


class EngineStepGraphs:
    """Stands in for ``BucketedCUDAGraphs`` (transcriber.py:31-173): ``forward(tokens, positions, slots)``
    replays the engine's captured decode step for that row count."""

    def __init__(self, model: B200Model):
        self.model = model
        self.hits, self.misses, self.buckets = defaultdict(int), 0, []

    def forward(self, tokens, positions, slot_indices):
        self.hits[int(tokens.shape[0])] += 1
        return self.model.decoder.forward_flash(tokens, None, None, positions, slot_indices=slot_indices)


def _slot_of(xa: torch.Tensor, xa_cache: torch.Tensor) -> int:
    """Slot whose row of ``xa_cache`` the view ``xa`` is (the Transcriber hands ``xa_cache[slot]`` around)."""
    if xa.untyped_storage().data_ptr() != xa_cache.untyped_storage().data_ptr():
        raise ValueError("word timing: the encoder states passed in are not a row of the transcriber's xa_cache")
    return (xa.storage_offset() - xa_cache.storage_offset()) // xa_cache.stride(0)


def make_fill_word_timings_batch(ref_dtw, original, xa_cache_of):
    """The replacement for ``fill_word_timings_batch``.  ``ref_dtw`` is the reference's ``dtw_align`` module:
    its text functions (``parse_predicted_lines``, ``chunk_speaker_lines``, ``_prepare_chunk``,
    ``rebuild_with_timings``) are called unchanged; only the decoder pass with hooks, ``_dtw_prep_batch`` and
    the numba DTW (dtw_align.py:1176-1238) are replaced by the engine.  Calls for any other model object
    go to ``original``."""

    def fill_word_timings_batch(model, tokenizer, slot_data, *, head_mask=None, max_tokens: int = 440):
        if not isinstance(model, B200Model):
            return original(model, tokenizer, slot_data, head_mask=head_mask, max_tokens=max_tokens)
        outs = [d[1] for d in slot_data]
        if not slot_data:
            return outs
        if head_mask is None:
            head_mask = ref_dtw.make_head_mask(model)
        heads = [tuple(int(v) for v in r) for r in head_mask.nonzero().tolist()]
        eng = model.engine
        if getattr(eng, "align_heads", None) != heads:
            eng.align_configure(heads)
        xa_cache = xa_cache_of(model)
        flats, recs, chunks, owners = [], [], [], []
        for si, (xa, pred_text, num_frames) in enumerate(slot_data):
            lines, flat, tag_anchors = ref_dtw.parse_predicted_lines(pred_text)
            flats.append(flat)
            if not flat:
                continue
            for ci, chunk_lines in enumerate(ref_dtw.chunk_speaker_lines(lines, tokenizer, max_tokens)):
                rec = ref_dtw._prepare_chunk(chunk_lines, tokenizer, flat, tag_anchors, max_tokens)
                if rec is None:
                    continue
                recs.append(rec)
                owners.append(si)
                chunks.append(alignment.AlignChunk(
                    slot=_slot_of(xa, xa_cache), ids=list(rec["ids"]),
                    word_lens=[len(t) for t in rec["ext_word_tokens"][:-1]], num_frames=int(num_frames),
                    word_anchors=rec.get("word_anchors") or [], tag_anchors=rec.get("tag_anchors") or []))
        if not chunks:
            return outs
        sot = tuple(tokenizer.sot_sequence)
        times = alignment.align_chunks(eng, chunks, sot_sequence=sot, no_timestamps=tokenizer.no_timestamps,
                                       eot=tokenizer.eot)
        # anchor stitching across the chunks of one window, as dtw_align.py:1240-1297
        out_t: dict[int, list] = {}
        prev_end: dict[int, float | None] = {}
        n_done: dict[int, int] = defaultdict(int)
        for rec, si, wt in zip(recs, owners, times):
            k = n_done[si]
            n_done[si] += 1
            if not wt:
                continue
            tagged, flat = rec["tagged"], flats[si]
            t_of = [wt[i] if i < len(wt) else None for i in range(len(tagged))]
            shift = 0.0
            if k > 0:
                anchor = next(((i, flat[oi][1]) for i, (oi, _) in enumerate(tagged)
                               if oi is not None and flat[oi][1] is not None and t_of[i] is not None), None)
                if anchor is not None:
                    shift = anchor[1] - t_of[anchor[0]][0]
                elif prev_end.get(si) is not None:
                    first = next((t_of[i] for i, (oi, _) in enumerate(tagged) if oi is not None and t_of[i] is not None),
                                 None)
                    shift = prev_end[si] - first[0] if first else 0.0
            dst = out_t.setdefault(si, [None] * len(flat))
            last = None
            for i, (oi, _) in enumerate(tagged):
                if oi is None or t_of[i] is None:
                    continue
                dst[oi] = (float(t_of[i][0]) + shift, float(t_of[i][1]) + shift)
                last = dst[oi][1]
            if last is not None:
                prev_end[si] = last
        for si, tt in out_t.items():
            outs[si] = ref_dtw.rebuild_with_timings(slot_data[si][1], flats[si], tt)
        return outs

    return fill_word_timings_batch


_XA_CACHES: dict[int, torch.Tensor] = {}     # id(B200Model) -> the xa_cache of the transcriber bound to it


def bind(transcriber, logmel: bool = True, word_timing: bool = True):
    """Completes the hand-over for a reference ``Transcriber`` built around a ``B200Model``; call it once,
    before the first ``transcribe``.  Loads the transcriber's device state (its ``load_model``), then swaps
    its CUDA-graph object and, optionally, its log-mel module and the word-timing function of its
    ``dtw_align`` module (calls for other models still reach the original function).  Returns the
    transcriber."""
    model = transcriber.model
    if not isinstance(model, B200Model):
        raise TypeError("dropin.bind expects a Transcriber whose model is a whisperdrz_b200.model.B200Model")
    model.skip_capture = True
    try:
        transcriber.load_model()
    finally:
        model.skip_capture = False
    transcriber.cuda_graphs = EngineStepGraphs(model)
    if logmel:
        transcriber.tomel = EngineLogMel(model, transcriber.tomel)
    if word_timing:
        pkg = type(transcriber).__module__.rsplit(".", 1)[0]
        ref_dtw = sys.modules.get(pkg + ".dtw_align")
        if ref_dtw is None:
            import importlib
            ref_dtw = importlib.import_module(pkg + ".dtw_align")
        _XA_CACHES[id(model)] = transcriber.xa_cache
        if not getattr(ref_dtw.fill_word_timings_batch, "_wdz_engine_binding", False):
            fn = make_fill_word_timings_batch(ref_dtw, ref_dtw.fill_word_timings_batch,
                                              lambda m: _XA_CACHES[id(m)])
            fn._wdz_engine_binding = True
            ref_dtw.fill_word_timings_batch = fn
    return transcriber
