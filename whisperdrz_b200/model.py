"""Drop-in model object for the reference's ``Transcriber(model=...)``.

The reference scheduler touches its model only through a small set of
attributes and methods (src/whisperdrz/transcriber.py:652-697, 1052-1108,
1676-1685): ``dims``, ``device``, ``dtype``, ``tokenizer``, ``cuda()``,
``encoder(mel)``, ``create_flash_kv``, ``reset_flash_kv``, ``prefill_flash``,
``decoder.cache_embedding_weight`` and ``decoder.forward_flash``, plus
``seq_lens`` of the first self-attention cache object.  ``B200Model`` offers
exactly that surface on top of the CUDA engine, so the reference's own
``decode_batch`` (regex classification, mask tables, Phase-4 corrections) keeps
running unchanged on the logits this returns.

Differences a maintainer should know: the KV caches live inside the engine
(one allocation per kind), so the per-layer cache objects returned by
``create_flash_kv`` are views for bookkeeping only; ``prefill_flash`` fills the
logits of the last prompt position only (the only one the reference reads,
transcriber.py:1109) and returns zeros elsewhere.  ``whisperdrz_b200.dropin.bind``
finishes the hand-over (engine log-mel, engine step graphs, word timing).
"""
from __future__ import annotations

import torch

from .dims import ModelDimensions
from .engine import Engine


class _KVView:
    """Stands in for one ``FlashKVCache`` (model.py:98-147)."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, seq_lens: torch.Tensor):
        self.k_cache, self.v_cache, self.seq_lens = k, v, seq_lens


class _Decoder:
    def __init__(self, owner: "B200Model"):
        self._o = owner
        self._emit_cache: dict[tuple[int, int], torch.Tensor] = {}

    def cache_embedding_weight(self, dtype=None) -> None:  # model.py:531-533: nothing to do, the head is tied in place
        return None

    def forward_flash(self, tokens, self_kv, cross_kv, positions, slot_indices=None, return_hidden_states=False):
        """model.py:570-617 for seq == 1 (the decode loop) or a prompt [B, P].

        seq == 1 runs the engine's captured decode step (``wdz_decode_step`` with no rules): the row
        positions are the slot lengths the engine keeps, which is what the reference passes
        (transcriber.py:1676: ``self_kv[0].seq_lens[active]``).  While the calling stream is being
        captured into a CUDA graph (the reference's ``BucketedCUDAGraphs``, transcriber.py:91-119) the
        same work is enqueued kernel by kernel on that stream from device-resident index tensors, with
        no host copy and no synchronisation, so the capture holds the whole step."""
        if return_hidden_states:
            raise NotImplementedError("hidden states are not exported by the engine")
        o = self._o
        eng = o.engine
        B, S = tokens.shape
        dev = tokens.device
        slots = torch.arange(B, device=dev) if slot_indices is None else slot_indices
        capturing = dev.type == "cuda" and torch.cuda.is_current_stream_capturing()
        if capturing and o.skip_capture:
            return torch.zeros(B, S, eng.dims.n_vocab, dtype=o.dtype, device=dev)
        if S == 1 and not capturing:
            _, logits = eng.decode_step(tokens.reshape(-1), slots, rules=None, want_logits=True)
            return logits.to(o.dtype).view(B, 1, -1)
        if positions.dim() == 1:
            positions = positions[:, None] + torch.arange(S, device=dev)[None]
        if S == 1:
            logits = eng.forward_rows(tokens.reshape(-1), slots, positions.reshape(-1))
            return logits.to(o.dtype).view(B, 1, -1)
        emit = self._emit_cache.get((B, S))
        if emit is None:
            emit = self._emit_cache[(B, S)] = torch.arange(S - 1, B * S, S, device=dev, dtype=torch.int32)
        logits = eng.forward_rows(tokens.reshape(-1), slots.repeat_interleave(S), positions.reshape(-1),
                                  emit_rows=emit)
        out = torch.zeros(B, S, eng.dims.n_vocab, dtype=o.dtype, device=dev)
        out[:, -1] = logits.to(o.dtype)
        return out


class B200Model:
    def __init__(self, dims: ModelDimensions, state_dict: dict, dtype=torch.bfloat16, device="cuda:0",
                 tokenizer=None, max_clips: int = 16):
        self.dims, self._sd, self._dtype = dims, state_dict, dtype
        self._device = torch.device(device)
        self._tokenizer = tokenizer
        self._max_clips = max_clips
        self.engine: Engine | None = None
        self.decoder = _Decoder(self)
        self.config = None
        # True while ``dropin.bind`` loads the reference Transcriber: graph captures of forward_flash then
        # record nothing, because bind replaces those graphs with the engine's own captured step
        self.skip_capture = False

    # attributes the Transcriber reads (transcriber.py:659-666)
    @property
    def device(self):
        return self._device

    @property
    def dtype(self):
        return self._dtype

    @property
    def tokenizer(self):
        if self._tokenizer is None:
            raise RuntimeError("pass tokenizer= (the reference's get_tokenizer(...)) to B200Model")
        return self._tokenizer

    def cuda(self):
        return self

    def eval(self):
        return self

    def create_flash_kv(self, batch_size: int, max_tokens: int | None = None):
        """model.py:773-811: builds the engine (it owns the caches) and returns per-layer views."""
        self.engine = Engine(self.dims, self._sd, dtype=self._dtype, device=self._device, n_slots=batch_size,
                             max_tokens=max_tokens or self.dims.n_text_ctx, max_clips=self._max_clips,
                             max_rows=max(64, batch_size * 8, self.dims.n_text_ctx))   # >= one alignment chunk
        e = self.engine
        L = self.dims.n_text_layer
        H = self.dims.n_text_head
        sv = lambda t: t.view(t.shape[0], t.shape[1], H, -1)
        self_kv = [_KVView(sv(e.self_k[l]), sv(e.self_v[l]), e.seq_lens_dev) for l in range(L)]
        cross_kv = [_KVView(sv(e.cross_k[l]), sv(e.cross_v[l]), e.seq_lens_dev) for l in range(L)]
        return self_kv, cross_kv

    def reset_flash_kv(self, self_kv, cross_kv, slot_indices=None):
        """model.py:813-822."""
        slots = range(self.engine.n_slots) if slot_indices is None else slot_indices
        self.engine.slot_reset(slots)

    def encoder(self, mel: torch.Tensor) -> torch.Tensor:
        """model.py:462-475; more than max_clips windows are encoded in groups."""
        outs = [self.engine.encode(mel[i: i + self._max_clips].float())
                for i in range(0, mel.shape[0], self._max_clips)]
        return torch.cat(outs, 0)

    def prefill_flash(self, tokens, xa, self_kv, cross_kv, slot_indices=None, return_hidden_states=False):
        """model.py:824-869."""
        B, P = tokens.shape
        slots = torch.arange(B, device=tokens.device) if slot_indices is None else slot_indices
        side = None
        if tokens.is_cuda:
            # The prompt rows share the decode step's scratch buffers.  When the caller prefills on a side stream
            # (the reference's warm slots, transcriber.py:976-994) the two streams are ordered around the call.
            cur, main = torch.cuda.current_stream(tokens.device), torch.cuda.default_stream(tokens.device)
            if cur != main:
                side = (cur, main)
        for i in range(0, B, self._max_clips):
            self.engine.cross_kv(xa[i: i + self._max_clips], slots[i: i + self._max_clips])
        self.engine.slot_reset(slots)
        pos = torch.zeros(B, dtype=torch.long, device=tokens.device)
        if side:
            side[0].wait_stream(side[1])
        out = self.decoder.forward_flash(tokens, self_kv, cross_kv, pos, slots, return_hidden_states)
        if side:
            side[1].wait_stream(side[0])
        return out
