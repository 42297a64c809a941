"""Continuous-batching scheduler and chunk-and-stitch front of the engine.

Mirrors the control flow of the reference ``Transcriber``
(src/whisperdrz/transcriber.py): ``transcribe(audio)`` splits audio into 30 s
chunks (:780-793), chunks wait in ``pending_chunks``, free slots are filled
and prefilled (:1555-1567, ``_init_slot`` :903-974, ``_prefill_slots``
:1042-1145), every loop iteration decodes one token for all started slots
(:1666-1744), finished slots are emitted and refilled at once (:1790-1815),
results are ordered by chunk id and joined (:803-810); ``__call__`` / ``flush``
give the pipeline form (:833-870, :1831-1844).

What changes is the device side of each step: one rule-descriptor upload, one
fused engine call (forward over all active rows, logit rules, argmax) and one
4-byte-per-row download replace the reference's ~30 mask kernels, bucketed
graph replay and six small copies.  Rules are the token-level subset of
``whisperdrz_b200.rules``; text-level rules and the text clean-up chain of the
reference are not part of this path.  Word timing by DTW on the alignment
heads (``_batch_align_slots`` :1419-1530) runs on every finished window when
an ``aligner`` is given (``whisperdrz_b200.alignment``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .dims import SAMPLE_RATE, TOK_EOT, TOK_LANG_EN, TOK_SOT, TOK_TRANSCRIBE
from .rules import BatchRuleState, segments as token_segments
from . import alignment


@dataclass
class TranscribeResults:
    """Same fields as the reference's TranscribeResults (transcriber.py:222-226)."""
    text: str
    raw_chunks: list | None = None
    segments: list | None = None


@dataclass
class Slot:
    index: int
    status: str = "ready"            # ready -> started -> finished -> ready (transcriber.py:505-509)
    chunk: dict | None = None
    last_token: int = 0
    stop_reason: str = ""
    win_offset: float = 0.0          # start of the current window inside the chunk, seconds
    continuations: int = 0
    kept_tokens: list = field(default_factory=list)     # tokens of earlier windows of this chunk
    kept_segments: list = field(default_factory=list)
    kept_words: list = field(default_factory=list)      # (token index in the chunk, start s, end s) of earlier windows
    window_words: list = field(default_factory=list)    # (token index in the window, start s, end s), chunk-relative times


def rules_to_array(rules: list[dict]) -> np.ndarray:
    """Rule dicts -> int32 [n, 32] in ``wdz_rule_desc`` layout."""
    a = np.zeros((len(rules), 32), dtype=np.int32)
    a[:, 0] = -1
    for i, r in enumerate(rules):
        if "forced_id" in r:
            a[i, 0] = r["forced_id"]
            continue
        a[i, 1] = r.get("mode", 0)
        a[i, 2] = r.get("arg0", 0)
        a[i, 3] = r.get("arg1", 0)
        a[i, 4] = np.int64(r.get("table_bits", 0)).astype(np.int32)
        a[i, 5] = r.get("prefix_begin", 0)
        a[i, 6] = r.get("prefix_end", 0)
        a[i, 14] = r.get("or_table", 0)
        a[i, 15] = r.get("allow_table", 0)
        for base, cap, key in ((7, 6, "set_ids"), (16, 4, "clear_ids"), (21, 10, "pen_ids")):
            ids = list(dict.fromkeys(r.get(key, ())))[:cap]
            a[i, base] = len(ids)
            a[i, base + 1: base + 1 + len(ids)] = ids
    return a


class Transcriber:
    def __init__(self, engine, BS: int | None = None, max_audio_length: float = 30.0,
                 max_new_tokens: int = 224, lang: str | None = "en", use_rules: bool = True,
                 text_decoder=None, max_continuations: int = 20, device_rules: bool | None = None,
                 steps_per_poll: int = 8, min_refill: int = 1, max_refill_wait: int = 4,
                 aligner=None, align_heads=None, n_warm: int = 0):
        """engine: ``whisperdrz_b200.engine.Engine`` (or an object with the same
        methods).  BS: concurrent slots, at most the engine's.  max_new_tokens:
        generated tokens per 30 s window before EOT is forced.  text_decoder:
        optional ``list[int] -> str`` (the tokenizer is not part of this path).
        max_continuations: a window that ran out of tokens before the end of its
        chunk is continued from its last closing timestamp, at most this many
        times (transcriber.py:1283-1334; 0 disables).  device_rules: keep the
        token-level rule state on the GPU and queue ``steps_per_poll`` decode
        steps per host round trip (default: on when the engine offers it).
        min_refill: while other slots are decoding, new chunks are admitted only
        when at least this many can be prefilled together (the encoder is far
        more efficient on a batch of windows), or after ``max_refill_wait``
        scheduler iterations; the reference refills one by one
        (transcriber.py:1790-1815, ``min_refill_batch = 1``), which is the default.
        n_warm: extra slots that are prefilled in the background (transcriber.py:559-568, 976-1040): while
        BS slots decode, up to n_warm more chunks have their log-mel, encoder and cross K/V computed on a side
        stream; a warm slot starts decoding as soon as its event has completed and a decode slot is free,
        paying only its prompt rows then.  BS + n_warm may not exceed the engine's slots.
        aligner: ``tokens -> [chunk dict]`` (see ``alignment.token_aligner``); when given, every finished
        window is aligned by DTW before its slot is released and results carry ``word_times``
        (the reference's ``dtw_align=True``).  align_heads: (layer, head) pairs, default the large-v3 set."""
        self.engine = engine
        self.n_warm = max(0, n_warm)
        self.BS = BS or (engine.n_slots - self.n_warm)
        if self.BS < 1 or self.BS + self.n_warm > engine.n_slots:
            raise ValueError("BS + n_warm exceeds the engine's slot count")
        self.max_audio_length = max_audio_length
        self.max_new_tokens = max_new_tokens
        self.use_rules = use_rules
        self.text_decoder = text_decoder
        self.max_continuations = max_continuations
        self.device_rules = (hasattr(engine, "ts_steps") and use_rules) if device_rules is None else device_rules
        self.steps_per_poll = max(1, steps_per_poll)
        self.min_refill, self.max_refill_wait = max(1, min_refill), max_refill_wait
        self._refill_waited = 0
        self._tok_cache: dict[int, list] = {}
        self.init_tokens = [TOK_SOT, TOK_LANG_EN, TOK_TRANSCRIBE] if lang else [TOK_SOT]
        if len(self.init_tokens) + max_new_tokens > engine.max_tokens:
            raise ValueError("prompt + max_new_tokens exceed the KV cache length")
        self.states = [Slot(i) for i in range(self.BS + self.n_warm)]
        self.rule_state = BatchRuleState(self.BS + self.n_warm, max_new_tokens)
        self.prefill_stream = None          # side stream of the warm slots, made on first use
        self.warming: list = []             # [(event, [slots], xa-free marker)] prefill groups in flight
        self.promoted = 0
        self.pending_chunks: list[dict] = []
        self.seconds_processed = 0.0
        self.steps = 0
        self.launch_rows = 0
        self.aligner = aligner
        self.windows_aligned = 0
        if aligner is not None:
            engine.align_configure(align_heads or alignment.ALIGNMENT_HEADS_LARGE_V3)

    # ------------------------------------------------------------------ public
    def transcribe(self, audio) -> TranscribeResults:
        """audio: 1-D float array/tensor at 16 kHz (host or device)."""
        if isinstance(audio, np.ndarray):
            audio = torch.from_numpy(audio)
        audio = audio.squeeze()
        chunk_len = int(self.max_audio_length * SAMPLE_RATE)
        for i, start in enumerate(range(0, len(audio), chunk_len)):
            end = min(start + chunk_len, len(audio))
            self.pending_chunks.append({"audio": audio[start:end], "id": f"chunk_{i}",
                                        "duration": (end - start) / SAMPLE_RATE, "offset": start / SAMPLE_RATE})
        results = []
        while self.pending_chunks or any(s.status != "ready" for s in self.states):
            r = self._run_batched_inference()
            if r:
                results.extend(r)
        return self.stitch(results)

    def stitch(self, results: list[dict]) -> TranscribeResults:
        results.sort(key=lambda r: int(str(r.get("id", "chunk_0")).split("_")[-1]))
        segs = [s for r in results for s in r["segments"]]
        text = "\n".join(r.get("prediction", "") for r in results) if self.text_decoder else ""
        return TranscribeResults(text=text, raw_chunks=results, segments=segs)

    def __call__(self, chunk):
        if isinstance(chunk, list):
            self.pending_chunks.extend(c for c in chunk if isinstance(c, dict))
        elif isinstance(chunk, dict):
            self.pending_chunks.append(chunk)
        ready = sum(1 for s in self.states if s.status == "ready")
        if self.pending_chunks and len(self.pending_chunks) >= ready:
            return self._run_batched_inference()
        return None

    def flush(self):
        while self.pending_chunks or any(s.status != "ready" for s in self.states):
            r = self._run_batched_inference()
            if r:
                yield from r

    # ---------------------------------------------------------------- internals
    def _init_slot(self, slot: Slot, chunk: dict) -> None:
        slot.chunk = chunk
        slot.status = "started"
        self.rule_state.reset(slot.index, self.max_new_tokens)
        slot.stop_reason = ""
        slot.win_offset, slot.continuations = 0.0, 0
        slot.kept_tokens, slot.kept_segments = [], []
        slot.kept_words, slot.window_words = [], []

    def _prefill_slots(self, slots: list[Slot]) -> None:
        """Log-mel + encoder + cross K/V + prompt for new slots, then their first token."""
        eng = self.engine
        for g0 in range(0, len(slots), eng.max_clips):
            grp = slots[g0: g0 + eng.max_clips]
            self._first_tokens(grp, self._encode_group(grp))

    def _encode_group(self, grp: list[Slot]):
        """Audio upload, log-mel, encoder and cross K/V of at most max_clips windows, on the current stream.
        Returns None, or the encoder states when the engine only offers the fused prefill call."""
        eng = self.engine
        dev = eng.device
        n = [min(len(s.chunk["audio"]), 480000) for s in grp]
        first = grp[0].chunk["audio"]
        if isinstance(first, torch.Tensor) and first.is_cuda:
            buf = torch.zeros(len(grp), 480000, dtype=torch.float32, device=dev)
            for i, s in enumerate(grp):
                buf[i, : n[i]] = s.chunk["audio"][: n[i]]
        elif dev.type == "cuda" and all(isinstance(s.chunk["audio"], torch.Tensor) and s.chunk["audio"].is_pinned()
                                        and s.chunk["audio"].dtype == torch.float32 for s in grp):
            # caller-pinned host audio goes to the device directly, one asynchronous copy per chunk
            buf = torch.zeros(len(grp), 480000, dtype=torch.float32, device=dev)
            for i, s in enumerate(grp):
                buf[i, : n[i]].copy_(s.chunk["audio"][: n[i]], non_blocking=True)
        else:
            host = self._staging(len(grp))
            for i, s in enumerate(grp):
                host[i, : n[i]] = torch.as_tensor(s.chunk["audio"][: n[i]], dtype=torch.float32)
                host[i, n[i]:] = 0.0
            buf = host.to(dev, non_blocking=True)
            if dev.type == "cuda":
                self._pin_busy[id(host)] = torch.cuda.Event()
                self._pin_busy[id(host)].record(torch.cuda.current_stream(dev))
        # a continuation window starts at its offset inside the chunk; the (max - 8) floor is still
        # taken over the whole chunk (transcriber.py:1062-1072)
        offs = [int(round(s.win_offset * 100)) for s in grp]
        mel = eng.logmel(buf, n_samples=n, frame_offset=offs if any(offs) else None)
        xa = eng.encode(mel)
        if hasattr(eng, "cross_kv") and hasattr(eng, "forward_rows"):
            eng.cross_kv(xa, [s.index for s in grp])
            return None
        return xa

    def _staging(self, rows: int) -> torch.Tensor:
        """A pinned host buffer for one group of windows whose previous upload has left it (two rotate, so that a
        side-stream upload in flight never makes the host wait on the decode stream)."""
        eng = self.engine
        pool = getattr(eng, "_pin_pool", None)
        if pool is None:
            pool = [torch.zeros(eng.max_clips, 480000, dtype=torch.float32) for _ in range(2)]
            if eng.device.type == "cuda":
                pool = [b.pin_memory() for b in pool]
            try:
                eng._pin_pool = pool
            except AttributeError:
                pass
            self._pin_busy, self._pin_next = {}, 0
        if not hasattr(self, "_pin_busy"):
            self._pin_busy, self._pin_next = {}, 0
        buf = pool[self._pin_next % len(pool)]
        self._pin_next += 1
        ev = self._pin_busy.pop(id(buf), None)
        if ev is not None:
            ev.synchronize()
        return buf[:rows]

    def _first_tokens(self, grp: list[Slot], xa=None) -> None:
        """Prompt rows of slots whose cross K/V are in place (or come with ``xa``), and their first token, on
        the current stream."""
        eng = self.engine
        cap = max(1, getattr(eng, "max_rows", 1 << 30) // max(1, len(self.init_tokens)))
        if len(grp) > cap:                 # more prompt rows than one forward call takes
            for i in range(0, len(grp), cap):
                self._first_tokens(grp[i: i + cap], None if xa is None else xa[i: i + cap])
            return
        ids = [s.index for s in grp]
        if xa is not None:
            logits = eng.prefill(xa, ids, [self.init_tokens] * len(grp))
        else:
            P = len(self.init_tokens)
            eng.slot_reset(ids)
            logits = eng.forward_rows(self.init_tokens * len(grp), [i for i in ids for _ in range(P)],
                                      list(range(P)) * len(grp), emit_rows=list(range(P - 1, P * len(grp), P)))
        if self.device_rules:
            eng.ts_reset(ids, [self.max_new_tokens] * len(ids))
            eng.ts_first(logits, ids)
        else:
            rules = self._rules_dev(self.rule_state.rules_array(ids)) if self.use_rules else None
            self._accept(grp, eng.rules_argmax(logits, rules).tolist())

    # ---- warm slots: prefill on a side stream (transcriber.py:976-1040)
    def _kick_off_async_prefill(self, grp: list[Slot]) -> None:
        dev = self.engine.device
        for s in grp:
            s.status = "warming"
        if dev.type != "cuda":
            self.warming.append((None, grp, self._encode_group(grp)))
            return
        if self.prefill_stream is None:
            self.prefill_stream = torch.cuda.Stream(dev)
        main = torch.cuda.current_stream(dev)
        self.prefill_stream.wait_stream(main)      # the slots' previous windows have been read (alignment)
        with torch.cuda.stream(self.prefill_stream):
            xa = self._encode_group(grp)
            ev = torch.cuda.Event()
            ev.record(self.prefill_stream)
        self.warming.append((ev, grp, xa))

    def _promote_warm_slots(self, room: int, must: bool) -> list[Slot]:
        """Starts decoding for warm slots whose prefill event has completed, oldest first, as far as ``room``
        decode slots are free.  ``must``: nothing else is decoding, so wait for the oldest group."""
        out: list[Slot] = []
        while self.warming and room > 0:
            ev, grp, xa = self.warming[0]
            if ev is not None:
                if not ev.query() and not (must and not out):
                    break
                torch.cuda.current_stream(self.engine.device).wait_event(ev)
            k = min(room, len(grp))
            now, rest = grp[:k], grp[k:]
            if rest:
                self.warming[0] = (ev, rest, None if xa is None else xa[k:])
            else:
                self.warming.pop(0)
            for s in now:
                s.status = "started"
            self._first_tokens(now, None if xa is None else xa[:k])
            room -= k
            out += now
            self.promoted += k
        return out

    def _fill_warm_slots(self) -> None:
        eng = self.engine
        while self.pending_chunks:
            n_warming = sum(len(g) for _, g, _ in self.warming)
            free = [s for s in self.states if s.status == "ready"]
            take = min(self.n_warm - n_warming, len(free), len(self.pending_chunks), eng.max_clips)
            if take <= 0:
                break
            grp = free[:take]
            for s in grp:
                self._init_slot(s, self.pending_chunks.pop(0))
            self._kick_off_async_prefill(grp)

    def _rules_dev(self, rules) -> torch.Tensor:
        """int32 [n, 32] descriptor array (or a list of rule dicts) -> device tensor."""
        a = rules if isinstance(rules, np.ndarray) else rules_to_array(rules)
        return torch.from_numpy(a).to(self.engine.device, non_blocking=False)

    def _accept(self, slots: list, toks: list) -> None:
        rs = self.rule_state
        done = rs.update([s.index for s in slots], toks)
        for s, t, d in zip(slots, toks, done):
            s.last_token = int(t)
            if d:
                s.status = "finished"
                s.stop_reason = "eot" if t == TOK_EOT else "nan_logits"
                if rs.n_new[s.index] > rs.max_new[s.index]:
                    s.stop_reason = "max_tokens"

    def _finish(self, slot: Slot) -> dict | None:
        """Emits a finished slot, or turns it into a continuation window (returns None)."""
        c = slot.chunk
        raw = self._tok_cache.pop(slot.index) if self.device_rules else self.rule_state.slot_tokens(slot.index)
        toks = [t for t in raw if t != TOK_EOT]
        base = c.get("offset", 0.0) + slot.win_offset
        segs = token_segments(toks, base)
        duration = c.get("duration", 0.0)
        if (slot.stop_reason == "max_tokens" and slot.continuations < self.max_continuations and segs
                and duration - (segs[-1]["end"] - c.get("offset", 0.0)) > 0.5):
            # out of tokens before the end of the chunk: keep everything up to the last closing
            # timestamp and decode a new window that starts there (at least 1 s further on)
            last_end = segs[-1]["end"] - base
            n_keep = 0
            closes = 0
            for i, t in enumerate(toks):
                if t >= 50365:
                    closes += 1
                    if closes == 2 * len(segs):
                        n_keep = i + 1
                        break
            slot.kept_words += [(len(slot.kept_tokens) + i, a, b) for i, a, b in slot.window_words if i < n_keep]
            slot.kept_tokens += toks[:n_keep]
            slot.kept_segments += segs
            slot.win_offset += max(last_end, 1.0)
            slot.continuations += 1
            self.rule_state.reset(slot.index, self.max_new_tokens)
            slot.status, slot.stop_reason = "continue", ""
            return None
        all_toks = slot.kept_tokens + toks
        res = {k: v for k, v in c.items() if k not in ("audio", "mel")}
        res.update(id=c["id"], tokens=all_toks, stop_reason=slot.stop_reason, windows=slot.continuations + 1,
                   segments=slot.kept_segments + segs)
        if self.aligner is not None:
            res["word_times"] = slot.kept_words + [(len(slot.kept_tokens) + i, a, b) for i, a, b in slot.window_words]
        if self.text_decoder:
            res["prediction"] = self.text_decoder(all_toks)
        self.seconds_processed += duration
        slot.status, slot.chunk = "ready", None
        slot.kept_tokens, slot.kept_segments = [], []
        slot.kept_words, slot.window_words = [], []
        return res

    def _align_finished(self, slots: list[Slot]) -> None:
        """DTW word timing of the windows that just finished, all in one batch, while their slots still hold
        the windows' cross keys (transcriber.py:1419-1530 runs the same step before a slot is re-used)."""
        chunks, owners = [], []
        for s in slots:
            raw = self._tok_cache[s.index] if self.device_rules else self.rule_state.slot_tokens(s.index)
            toks = [t for t in raw if t != TOK_EOT]
            s.window_words = []
            c = s.chunk
            left = max(0.0, c.get("duration", self.max_audio_length) - s.win_offset)
            frames = int(min(self.max_audio_length, left) * alignment.FRAMES_PER_SECOND)
            for rec in self.aligner(toks):
                chunks.append(alignment.AlignChunk(slot=s.index, ids=rec["ids"], word_lens=rec["word_lens"], num_frames=frames,
                                                   word_anchors=rec.get("word_anchors", []), tag_anchors=rec.get("tag_anchors", [])))
                owners.append((s, rec["token_pos"]))
        if not chunks:
            return
        times = alignment.align_chunks(self.engine, chunks)
        self.windows_aligned += len(slots)
        for (s, pos), wt in zip(owners, times):
            base = s.chunk.get("offset", 0.0) + s.win_offset
            s.window_words += [(p, round(a + base, 2), round(b + base, 2)) for p, (a, b) in zip(pos, wt)]

    @torch.inference_mode()
    def step(self) -> list[dict]:
        """One scheduler iteration (the loop body of transcriber.py:1584-1815):
        refill free slots from ``pending_chunks`` and prefill them, decode one
        token for every started slot, emit the slots that finished."""
        eng = self.engine
        done: list[dict] = []
        new = []
        cont = [s for s in self.states if s.status == "continue"]
        if self.n_warm > 0:
            # continuation windows are prefilled in place; new chunks only enter through the warm pool
            for s in cont:
                s.status = "started"
            if cont:
                self._prefill_slots(cont)
            started = sum(1 for s in self.states if s.status == "started")
            self._promote_warm_slots(self.BS - started, must=started == 0)
            self._fill_warm_slots()
            started = sum(1 for s in self.states if s.status == "started")
            if started == 0 and self.warming:
                self._promote_warm_slots(self.BS, must=True)
        else:
            free = [s for s in self.states if s.status == "ready"]
            busy = any(s.status == "started" for s in self.states)
            n_admit = min(len(free), len(self.pending_chunks))
            if n_admit and busy and len(cont) + n_admit < self.min_refill and self._refill_waited < self.max_refill_wait:
                self._refill_waited += 1          # let a larger prefill batch build up while the others decode
                n_admit, cont = 0, []
            else:
                self._refill_waited = 0
            for s in cont:
                s.status = "started"
                new.append(s)
            for s in free[:n_admit]:
                self._init_slot(s, self.pending_chunks.pop(0))
                new.append(s)
            if new:
                self._prefill_slots(new)
        active = [s for s in self.states if s.status == "started"]
        if active and self.device_rules:
            # several steps per host round trip: rules, argmax and state updates all stay on the GPU
            ids = [s.index for s in active]
            eng.ts_steps(ids, self.steps_per_poll)
            self.steps += self.steps_per_poll
            self.launch_rows += len(active) * self.steps_per_poll
            st = eng.ts_poll()
            for s in active:
                row = st[s.index]
                if row[6]:                                   # done
                    n_new, max_new = int(row[1]), int(row[0])
                    toks = eng.ts_tokens(s.index, n_new)
                    self._tok_cache[s.index] = toks
                    s.status = "finished"
                    last = toks[-1] if toks else TOK_EOT
                    s.stop_reason = "max_tokens" if n_new > max_new else ("eot" if last == TOK_EOT else "nan_logits")
        elif active:
            ids = [s.index for s in active]
            rules = self._rules_dev(self.rule_state.rules_array(ids)) if self.use_rules else None
            nxt = eng.decode_step([s.last_token for s in active], ids, rules=rules)
            self.steps += 1
            self.launch_rows += len(active)
            self._accept(active, nxt.tolist())
            eng.device_status()          # a kernel that gave up (bounded wait, NaN row) must not pass for a token
        if self.aligner is not None:
            fin = [s for s in self.states if s.status == "finished"]
            if fin:
                # the alignment pass borrows the encoder's activation workspace: keep it apart from a
                # warm-slot encoder run on the side stream
                if self.prefill_stream is not None:
                    torch.cuda.current_stream(eng.device).wait_stream(self.prefill_stream)
                self._align_finished(fin)
                if self.prefill_stream is not None:
                    self.prefill_stream.wait_stream(torch.cuda.current_stream(eng.device))
        for s in self.states:
            if s.status == "finished":
                r = self._finish(s)
                if r is not None:
                    done.append(r)
        return done

    def busy(self) -> bool:
        return bool(self.pending_chunks) or any(s.status != "ready" for s in self.states)

    def _run_batched_inference(self):
        """Drains everything that is pending or in flight (transcriber.py:1532-1829)."""
        done: list[dict] = []
        while self.busy():
            done.extend(self.step())
        return done or None
