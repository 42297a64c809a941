"""Python host of the CUDA engine: owns the device tensors (torch is the
allocator), lends them to libwdz.so through the C ABI and exposes the engine
calls with torch tensors in and out.  Requires a CUDA device; there is no
fallback."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import capi, frontend
from .dims import ModelDimensions

_TORCH_DTYPE = {torch.float32: capi.WDZ_F32, torch.bfloat16: capi.WDZ_BF16}


def pack_weights(sd: dict, dims: ModelDimensions, dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """Reference state_dict (model.py names) -> the tensors the engine binds:
    q/k/v stacked per attention (key bias = 0, model.py:259), conv kernels
    tap-major ([out, tap * in + c]), cross-attention K/V projections of all
    decoder layers stacked into one [L * 2 * d, d] operand."""
    out: dict[str, torch.Tensor] = {}

    def put(name, t, dt=dtype):
        out[name] = t.detach().to(device=device, dtype=dt).contiguous()

    put("encoder.conv1.weight", sd["encoder.conv1.weight"].permute(0, 2, 1).reshape(dims.n_audio_state, -1))
    put("encoder.conv1.bias", sd["encoder.conv1.bias"])
    put("encoder.conv2.weight", sd["encoder.conv2.weight"].permute(0, 2, 1).reshape(dims.n_audio_state, -1))
    put("encoder.conv2.bias", sd["encoder.conv2.bias"])
    put("encoder.positional_embedding", sd["encoder.positional_embedding"], torch.float32)
    put("encoder.ln_post.weight", sd["encoder.ln_post.weight"])
    put("encoder.ln_post.bias", sd["encoder.ln_post.bias"])

    def block(p, cross):
        q, k, v = (sd[f"{p}.attn.{n}.weight"] for n in ("query", "key", "value"))
        put(f"{p}.attn.qkv.weight", torch.cat([q, k, v], 0))
        qb, vb = sd[f"{p}.attn.query.bias"], sd[f"{p}.attn.value.bias"]
        put(f"{p}.attn.qkv.bias", torch.cat([qb, torch.zeros_like(qb), vb], 0))
        names = ["attn_ln.weight", "attn_ln.bias", "attn.out.weight", "attn.out.bias", "mlp_ln.weight",
                 "mlp_ln.bias", "mlp.0.weight", "mlp.0.bias", "mlp.2.weight", "mlp.2.bias"]
        if cross:
            names += ["cross_attn_ln.weight", "cross_attn_ln.bias", "cross_attn.query.weight",
                      "cross_attn.query.bias", "cross_attn.out.weight", "cross_attn.out.bias"]
        for n in names:
            put(f"{p}.{n}", sd[f"{p}.{n}"])

    for i in range(dims.n_audio_layer):
        block(f"encoder.blocks.{i}", False)
    for i in range(dims.n_text_layer):
        block(f"decoder.blocks.{i}", True)
    put("decoder.token_embedding.weight", sd["decoder.token_embedding.weight"])
    put("decoder.positional_embedding", sd["decoder.positional_embedding"])
    put("decoder.ln.weight", sd["decoder.ln.weight"])
    put("decoder.ln.bias", sd["decoder.ln.bias"])
    kvw, kvb = [], []
    for i in range(dims.n_text_layer):
        p = f"decoder.blocks.{i}.cross_attn"
        kvw += [sd[f"{p}.key.weight"], sd[f"{p}.value.weight"]]
        kvb += [torch.zeros_like(sd[f"{p}.value.bias"]), sd[f"{p}.value.bias"]]
    put("decoder.cross_kv.weight", torch.cat(kvw, 0))
    put("decoder.cross_kv.bias", torch.cat(kvb, 0))
    return out


def pack_rules(rules: list[dict]) -> np.ndarray:
    """list of rule dicts -> array of ``wdz_rule_desc`` (uint8 [n, 128])."""
    arr = (capi.RuleDesc * max(len(rules), 1))()
    for i, r in enumerate(rules):
        d = arr[i]
        d.forced_id = r.get("forced_id", -1)
        d.mode = r.get("mode", capi.MODE_OR)
        d.arg0, d.arg1 = r.get("arg0", 0), r.get("arg1", 0)
        d.table_bits = r.get("table_bits", 0)
        d.prefix_begin, d.prefix_end = r.get("prefix_begin", 0), r.get("prefix_end", 0)
        d.or_table, d.allow_table = r.get("or_table", 0), r.get("allow_table", 0)
        for field, cap in (("set_ids", 6), ("clear_ids", 4), ("pen_ids", 10)):
            ids = list(dict.fromkeys(r.get(field, [])))
            if len(ids) > cap:
                raise ValueError(f"rule {i}: {len(ids)} {field} > {cap}")
            setattr(d, "n_" + field.split("_")[0], len(ids))
            for j, t in enumerate(ids):
                getattr(d, field)[j] = int(t)
    return np.frombuffer(bytes(arr), dtype=np.uint8).reshape(-1, 128)[: len(rules)].copy()


def pack_tables(tables: torch.Tensor, n_vocab: int) -> torch.Tensor:
    """bool [n_tables, V] -> uint32 bitsets as int32 tensor [max(n_tables, 32), ceil(V / 32)]."""
    words = (n_vocab + 31) // 32
    n = max(capi.MAX_TABLES, int(tables.shape[0]))
    t = np.zeros((n, words * 32), dtype=np.uint8)
    tb = tables.cpu().numpy().astype(np.uint8)
    t[: tb.shape[0], :n_vocab] = tb
    packed = np.packbits(t.reshape(n, words, 32), axis=-1, bitorder="little")
    return torch.from_numpy(packed.view(np.uint32).reshape(n, words).view(np.int32).copy())


class Engine:
    """One engine per GPU per process (the C library is not thread-safe)."""

    def __init__(self, dims: ModelDimensions, state_dict: dict, dtype: torch.dtype = torch.bfloat16,
                 device: str | torch.device = "cuda:0", n_slots: int = 32, max_tokens: int | None = None,
                 max_clips: int = 16, max_rows: int | None = None, flags: int = 0,
                 tables: torch.Tensor | None = None, lend_workspace: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("whisperdrz_b200.Engine needs a CUDA device (no CPU path exists)")
        if dtype not in _TORCH_DTYPE:
            raise ValueError("dtype must be torch.float32 or torch.bfloat16")
        self.lib = capi.load()
        self.dims, self.dtype = dims, dtype
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.n_slots = n_slots
        self.max_tokens = max_tokens or dims.n_text_ctx
        self.max_clips = max_clips
        self.max_rows = max_rows or max(n_slots, 64)
        cfg = capi.Config(*[getattr(dims, f) for f in (
            "n_mels", "n_audio_ctx", "n_audio_state", "n_audio_head", "n_audio_layer",
            "n_vocab", "n_text_ctx", "n_text_state", "n_text_head", "n_text_layer")],
            _TORCH_DTYPE[dtype], n_slots, self.max_tokens, max_clips, self.max_rows, flags)
        self.cfg = cfg
        h = C.c_void_p()
        rc = self.lib.wdz_engine_create(C.byref(cfg), C.byref(h))
        if rc != capi.WDZ_OK:
            raise capi.WdzError(rc, "wdz_engine_create rejected the configuration")
        self.h = h
        dev = self.device
        self.weights = pack_weights(state_dict, dims, dtype, dev)
        L, d = dims.n_text_layer, dims.n_text_state
        self.self_k = torch.zeros(L, n_slots, self.max_tokens, d, dtype=dtype, device=dev)
        self.self_v = torch.zeros_like(self.self_k)
        self.cross_k = torch.zeros(L, n_slots, dims.n_audio_ctx, d, dtype=dtype, device=dev)
        self.cross_v = torch.zeros_like(self.cross_k)
        self.seq_lens_dev = torch.zeros(n_slots, dtype=torch.int32, device=dev)
        fb, lo, hi = frontend.mel_filterbank(dims.n_mels)
        self.consts = {
            "mel.twiddle": torch.from_numpy(frontend.twiddle()).to(dev),
            "mel.window": torch.from_numpy(frontend.hann_periodic()).to(dev),
            "mel.fb": torch.from_numpy(fb).to(dev),
            "mel.band_lo": torch.from_numpy(lo).to(dev),
            "mel.band_hi": torch.from_numpy(hi).to(dev),
        }
        self.tables_dev = None
        if tables is not None:
            self.tables_dev = pack_tables(tables, dims.n_vocab).to(dev)
        for name, t in self.weights.items():
            self._bind(name, t)
        for name, t in self.consts.items():
            self._bind(name, t)
        for name, t in (("cache.self_k", self.self_k), ("cache.self_v", self.self_v),
                        ("cache.cross_k", self.cross_k), ("cache.cross_v", self.cross_v),
                        ("cache.seq_lens", self.seq_lens_dev)):
            self._bind(name, t)
        if self.tables_dev is not None:
            self._bind("rules.tables", self.tables_dev)
        # lend_workspace=False: a host with no scratch memory to give; only the entry points that bring their own
        # scratch (logmel_static) work then, the others answer WDZ_ENOMEM
        self.workspace = None
        if lend_workspace:
            need = C.c_size_t()
            self._check(self.lib.wdz_workspace_bytes(self.h, C.byref(need)))
            self.workspace = torch.empty(need.value, dtype=torch.uint8, device=dev)
            self._check(self.lib.wdz_set_workspace(self.h, self.workspace.data_ptr(), need.value))
        self._check(self.lib.wdz_finalize(self.h))

    # ------------------------------------------------------------------ util
    def _bind(self, name: str, t: torch.Tensor) -> None:
        assert t.is_cuda and t.is_contiguous()
        self._check(self.lib.wdz_bind(self.h, name.encode(), t.data_ptr(), t.numel()))

    def _check(self, rc: int) -> None:
        if rc != capi.WDZ_OK:
            raise capi.WdzError(rc, self.lib.wdz_last_error(self.h).decode())

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _i32(self, x) -> torch.Tensor:
        if isinstance(x, torch.Tensor):
            return x.to(device=self.device, dtype=torch.int32).contiguous()
        return torch.tensor(list(x), dtype=torch.int32, device=self.device)

    def close(self) -> None:
        if getattr(self, "h", None):
            torch.cuda.synchronize(self.device)
            self.lib.wdz_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def device_status(self) -> None:
        """Raises if a kernel flagged an error (NaN logits row, exhausted wait)."""
        self._check(self.lib.wdz_device_status(self.h, self._stream()))

    # ----------------------------------------------------------- measurement
    def launch_count(self) -> int:
        out = C.c_int64()
        self._check(self.lib.wdz_launch_count(self.h, C.byref(out)))
        return out.value

    def profile(self, enable: bool) -> None:
        self._check(self.lib.wdz_profile(self.h, int(enable)))

    def profile_read(self) -> dict:
        """{kind: {"ms", "launches", "work"}} for the launches recorded since profile(True)."""
        res = {}
        for name, kind in capi.PROF_KINDS.items():
            ms, n, work = C.c_double(), C.c_int64(), C.c_double()
            self._check(self.lib.wdz_profile_read(self.h, kind, C.byref(ms), C.byref(n), C.byref(work)))
            res[name] = {"ms": ms.value, "launches": n.value, "work": work.value}
        return res

    # ------------------------------------------------------------- front end
    def _checked_lengths(self, N: int, B: int, n_samples) -> torch.Tensor:
        """Per-clip sample counts as a device tensor; lengths that come from the host are validated there, so that
        the call does not have to wait for the GPU (a device tensor is read back once)."""
        if n_samples is None:
            shortest, ns = N, self._i32([N] * B)
        elif isinstance(n_samples, torch.Tensor):
            ns = self._i32(n_samples)
            shortest = int(ns.min())
        else:
            host = [int(v) for v in n_samples]
            shortest, ns = min(host), self._i32(host)
        if shortest < 400:
            raise ValueError("clips shorter than 400 samples cannot be reflect-padded")
        return ns

    def logmel(self, audio: torch.Tensor, n_samples=None, frame_offset=None) -> torch.Tensor:
        """audio f32 [B, N] (device) -> mel f32 [B, n_mels, 3000]."""
        audio = audio.to(device=self.device, dtype=torch.float32)
        if audio.dim() == 1:
            audio = audio[None]
        audio = audio.contiguous()
        B, N = audio.shape
        if N > 480000:
            raise ValueError("a window holds at most 30 s (480000 samples)")
        ns = self._checked_lengths(N, B, n_samples)
        fo = None if frame_offset is None else self._i32(frame_offset)
        mel = torch.empty(B, self.dims.n_mels, 3000, dtype=torch.float32, device=self.device)
        self._check(self.lib.wdz_logmel(self.h, audio.data_ptr(), N, ns.data_ptr(),
                                        None if fo is None else fo.data_ptr(), B, mel.data_ptr(), self._stream()))
        return mel

    def logmel_static(self, audio: torch.Tensor, n_samples=None, frame_offset=None) -> torch.Tensor:
        """``logmel`` through the entry point that brings its own scratch: for
        embedders that cannot lend the engine a workspace (all GPU memory
        already handed to another pool, or no tolerance for the stall of a
        device allocation).  At most 4 clips per call; calls share one built-in
        array, so do not overlap them on the GPU; make the first call on a
        device before any stream capture."""
        audio = audio.to(device=self.device, dtype=torch.float32)
        if audio.dim() == 1:
            audio = audio[None]
        audio = audio.contiguous()
        B, N = audio.shape
        if N > 480000:
            raise ValueError("a window holds at most 30 s (480000 samples)")
        ns = self._checked_lengths(N, B, n_samples)
        fo = None if frame_offset is None else self._i32(frame_offset)
        mel = torch.empty(B, self.dims.n_mels, 3000, dtype=torch.float32, device=self.device)
        self._check(self.lib.wdz_logmel_static(self.h, audio.data_ptr(), N, ns.data_ptr(),
                                               None if fo is None else fo.data_ptr(), B, mel.data_ptr(),
                                               self._stream()))
        return mel

    # --------------------------------------------------------------- encoder
    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        mel = mel.to(device=self.device, dtype=torch.float32).contiguous()
        B = mel.shape[0]
        assert mel.shape[1:] == (self.dims.n_mels, 2 * self.dims.n_audio_ctx), mel.shape
        xa = torch.empty(B, self.dims.n_audio_ctx, self.dims.n_audio_state, dtype=self.dtype, device=self.device)
        self._check(self.lib.wdz_encode(self.h, mel.data_ptr(), B, xa.data_ptr(), self._stream()))
        return xa

    def linear(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gelu: bool = False,
               cuda_cores_only: bool | int = False) -> torch.Tensor:
        """act(x @ w.T + bias) in the engine dtype through the engine's GEMM kernels (``cuda_cores_only``: True/1 =
        no tensor cores, 2 = the lone-CTA tcgen05 kernel, no CTA pairs)."""
        x = x.to(device=self.device, dtype=self.dtype).contiguous()
        w = w.to(device=self.device, dtype=self.dtype).contiguous()
        b = None if bias is None else bias.to(device=self.device, dtype=self.dtype).contiguous()
        M, K = x.shape
        N = w.shape[0]
        y = torch.empty(M, N, dtype=self.dtype, device=self.device)
        self._check(self.lib.wdz_linear(self.h, x.data_ptr(), M, K, w.data_ptr(), None if b is None else b.data_ptr(),
                                        N, int(gelu), y.data_ptr(), int(cuda_cores_only), self._stream()))
        return y

    def linear_rows(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        """Decode-shaped product: x [M, K] (engine dtype) @ w[N, K].T (+ bias) -> f32 [M, N];
        with ``out`` given the result is added into it."""
        x = x.to(device=self.device, dtype=self.dtype).contiguous()
        w = w.to(device=self.device, dtype=self.dtype).contiguous()
        b = None if bias is None else bias.to(device=self.device, dtype=self.dtype).contiguous()
        M, K = x.shape
        N = w.shape[0]
        y = out if out is not None else torch.empty(M, N, dtype=torch.float32, device=self.device)
        self._check(self.lib.wdz_linear_rows(self.h, x.data_ptr(), M, K, w.data_ptr(),
                                             None if b is None else b.data_ptr(), N, int(out is not None),
                                             y.data_ptr(), self._stream()))
        return y

    def encoder_attention(self, qkv: torch.Tensor, cuda_cores_only: bool = False) -> torch.Tensor:
        """qkv [B, n_audio_ctx, 3d] -> [B, n_audio_ctx, d] (non-causal, scale 1/8) in the engine dtype."""
        qkv = qkv.to(device=self.device, dtype=self.dtype).contiguous()
        B, T, d3 = qkv.shape
        assert T == self.dims.n_audio_ctx and d3 == 3 * self.dims.n_audio_state and B <= self.max_clips
        out = torch.empty(B, T, d3 // 3, dtype=self.dtype, device=self.device)
        self._check(self.lib.wdz_encoder_attention(self.h, qkv.data_ptr(), B, out.data_ptr(), int(cuda_cores_only),
                                                   self._stream()))
        return out

    # --------------------------------------------------------------- decoder
    def cross_kv(self, xa: torch.Tensor, slots) -> None:
        xa = xa.to(self.dtype).contiguous()
        s = self._i32(slots)
        self._check(self.lib.wdz_cross_kv(self.h, xa.data_ptr(), s.data_ptr(), xa.shape[0], self._stream()))

    def slot_reset(self, slots) -> None:
        s = self._i32(slots)
        self._check(self.lib.wdz_slot_reset(self.h, s.data_ptr(), s.numel(), self._stream()))

    def seq_lens(self) -> list[int]:
        out = (C.c_int32 * self.n_slots)()
        self._check(self.lib.wdz_slot_seqlens(self.h, out, self._stream()))
        return list(out)

    def forward_rows(self, tokens, slots, positions, emit_rows=None, want_logits: bool = True):
        t, s, p = self._i32(tokens), self._i32(slots), self._i32(positions)
        n = t.numel()
        er = None if emit_rows is None else self._i32(emit_rows)
        n_emit = n if er is None else er.numel()
        logits = None
        if want_logits:
            logits = torch.empty(n_emit, self.dims.n_vocab, dtype=torch.float32, device=self.device)
        self._check(self.lib.wdz_forward_rows(
            self.h, t.data_ptr(), s.data_ptr(), p.data_ptr(), n, None if er is None else er.data_ptr(), n_emit,
            None if logits is None else logits.data_ptr(), self._stream()))
        return logits

    def prefill(self, xa: torch.Tensor, window_slots, prompts: list[list[int]], want_logits: bool = True):
        """Cross K/V + slot reset + prompt rows; returns the logits of each
        window's last prompt token, f32 [B, V]."""
        xa = xa.to(self.dtype).contiguous()
        ws = self._i32(window_slots)
        slots_l = [int(v) for v in ws.tolist()]
        tok, sl, pos, emit = [], [], [], []
        for b, pr in enumerate(prompts):
            for j, t in enumerate(pr):
                tok.append(int(t)); sl.append(slots_l[b]); pos.append(j)
            emit.append(len(tok) - 1)
        t, s, p, er = self._i32(tok), self._i32(sl), self._i32(pos), self._i32(emit)
        logits = None
        if want_logits:
            logits = torch.empty(len(emit), self.dims.n_vocab, dtype=torch.float32, device=self.device)
        self._check(self.lib.wdz_prefill(
            self.h, xa.data_ptr(), ws.data_ptr(), xa.shape[0], t.data_ptr(), s.data_ptr(), p.data_ptr(), t.numel(),
            er.data_ptr(), er.numel(), None if logits is None else logits.data_ptr(), self._stream()))
        return logits

    def rules_to_device(self, rules) -> torch.Tensor | None:
        if rules is None:
            return None
        if isinstance(rules, torch.Tensor):
            return rules
        return torch.from_numpy(pack_rules(rules)).to(self.device)

    def decode_step(self, tokens, slots, rules=None, want_logits: bool = False):
        """One step for the given (last token, slot) rows; returns next ids
        (int32, device) and optionally the f32 logits."""
        t, s = self._i32(tokens), self._i32(slots)
        n = t.numel()
        rd = self.rules_to_device(rules)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        logits = torch.empty(n, self.dims.n_vocab, dtype=torch.float32, device=self.device) if want_logits else None
        self._check(self.lib.wdz_decode_step(
            self.h, t.data_ptr(), s.data_ptr(), n, None if rd is None else rd.data_ptr(), out.data_ptr(),
            None if logits is None else logits.data_ptr(), self._stream()))
        return (out, logits) if want_logits else out

    # ------------------------------------------- rule state kept on the device
    def ts_reset(self, slots, max_new) -> None:
        s, m = self._i32(slots), self._i32(max_new)
        self._check(self.lib.wdz_ts_reset(self.h, s.data_ptr(), m.data_ptr(), s.numel(), self._stream()))

    def ts_first(self, logits: torch.Tensor, slots) -> None:
        logits = logits.to(device=self.device, dtype=torch.float32).contiguous()
        s = self._i32(slots)
        self._check(self.lib.wdz_ts_first(self.h, logits.data_ptr(), s.data_ptr(), s.numel(), self._stream()))

    def ts_steps(self, slots, k: int) -> None:
        s = self._i32(slots)
        self._check(self.lib.wdz_ts_steps(self.h, s.data_ptr(), s.numel(), int(k), self._stream()))

    def ts_poll(self) -> np.ndarray:
        """int32 [n_slots, 24]: max_new, n_new, timing_count, last_timing, last_was_timing, n_recent, done,
        last_token, recent[10], spare[6]."""
        out = np.empty((self.n_slots, 24), dtype=np.int32)
        self._check(self.lib.wdz_ts_poll(self.h, out.ctypes.data, self._stream()))
        return out

    def ts_tokens(self, slot: int, n: int) -> list[int]:
        out = np.empty(max(n, 1), dtype=np.int32)
        self._check(self.lib.wdz_ts_tokens(self.h, int(slot), out.ctypes.data, int(n), self._stream()))
        return out[:n].tolist()

    def reargmax(self, rows, rules) -> torch.Tensor:
        r = self._i32(rows)
        rd = self.rules_to_device(rules)
        out = torch.empty(r.numel(), dtype=torch.int32, device=self.device)
        self._check(self.lib.wdz_reargmax(self.h, r.data_ptr(), None if rd is None else rd.data_ptr(), r.numel(),
                                          out.data_ptr(), self._stream()))
        return out

    def rules_argmax(self, logits: torch.Tensor, rules, penalty: bool = True) -> torch.Tensor:
        logits = logits.to(device=self.device, dtype=torch.float32).contiguous()
        rd = self.rules_to_device(rules)
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        self._check(self.lib.wdz_rules_argmax(self.h, logits.data_ptr(), None if rd is None else rd.data_ptr(),
                                              logits.shape[0], int(penalty), out.data_ptr(), self._stream()))
        return out

    # ------------------------------------------------------- word-timing alignment
    def align_configure(self, heads) -> None:
        """(layer, head) pairs whose cross-attention tracks time (dtw_align.py:52-62)."""
        arr = np.ascontiguousarray(np.asarray(heads, dtype=np.int32).reshape(-1, 2))
        self._check(self.lib.wdz_align_configure(self.h, arr.ctypes.data, arr.shape[0]))
        self.align_heads = [tuple(int(v) for v in r) for r in arr]

    def align_capacity(self, t_pad: int) -> int:
        return int(self.lib.wdz_align_capacity(self.h, int(t_pad)))

    def align_matrix(self, tokens, lens, slots, audio_caps) -> torch.Tensor:
        """tokens int [B, T] (``alignment.build_full_tokens``), lens / slots / audio_caps [B] ->
        f32 [B, T, n_audio_ctx] on the device: the cost matrix before negation, rows past a chunk's length
        zero (dtw_align.py:1181-1195).  Slots must be distinct; more chunks than one call takes are run
        in several calls."""
        tok = torch.as_tensor(np.asarray(tokens), dtype=torch.int32)
        B, T = tok.shape
        if len(set(int(s) for s in slots)) != B:
            raise ValueError("align_matrix: the chunks of one call must sit in distinct slots")
        out = torch.empty(B, T, self.dims.n_audio_ctx, dtype=torch.float32, device=self.device)
        cap = self.align_capacity(T)
        if cap < 1:
            raise capi.WdzError(-5, f"no room to align chunks of {T} tokens (configure heads first)")
        tok_d = tok.to(self.device)
        lens_d, slots_d, caps_d = self._i32(lens), self._i32(slots), self._i32(audio_caps)
        for b0 in range(0, B, cap):
            n = min(cap, B - b0)
            self._check(self.lib.wdz_align_matrix(
                self.h, tok_d[b0:b0 + n].contiguous().data_ptr(), lens_d[b0:].data_ptr(), slots_d[b0:].data_ptr(),
                caps_d[b0:].data_ptr(), n, T, out[b0:].data_ptr(), self._stream()))
        return out

    def dtw(self, matrix: torch.Tensor, row0, n_rows, n_cols, limits=None):
        """Minimum-cost monotonic paths through ``-matrix[b, row0[b] : row0[b] + n_rows[b], : n_cols[b]]``
        (dtw_align.py:170-223).  ``limits`` = per chunk (lo, hi) int arrays [n_rows[b]]: columns outside
        [lo, hi) of a row cost +inf (anchor bands, dtw_align.py:589-641).  Returns [(text_idx, time_idx)]
        as int64 numpy arrays."""
        matrix = matrix.to(device=self.device, dtype=torch.float32)
        if matrix.dim() == 2:
            matrix = matrix[None]
        matrix = matrix.contiguous()
        B = matrix.shape[0]
        max_rows, max_cols = max(1, max(n_rows)), max(1, max(n_cols))
        lo_d = hi_d = None
        if limits is not None:
            lo = np.zeros((B, max_rows), dtype=np.int32)
            hi = np.zeros((B, max_rows), dtype=np.int32)
            for b, (l, h) in enumerate(limits):
                lo[b, : len(l)] = l
                hi[b, : len(h)] = h
            lo_d, hi_d = torch.from_numpy(lo).to(self.device), torch.from_numpy(hi).to(self.device)
        cap = max_rows + max_cols
        ti = torch.empty(B, cap, dtype=torch.int32, device=self.device)
        tj = torch.empty(B, cap, dtype=torch.int32, device=self.device)
        ln = torch.empty(B, dtype=torch.int32, device=self.device)
        row0_d, rows_d, cols_d = self._i32(row0), self._i32(n_rows), self._i32(n_cols)   # kept alive past the launch
        if min(int(r) for r in row0) < 0 or max(int(r) + int(n) for r, n in zip(row0, n_rows)) > matrix.shape[1] \
                or max_cols > matrix.shape[2]:
            raise ValueError("dtw: a chunk's rows or columns lie outside the matrix")
        self._check(self.lib.wdz_dtw(
            self.h, matrix.data_ptr(), matrix.stride(0), matrix.stride(1), row0_d.data_ptr(),
            rows_d.data_ptr(), cols_d.data_ptr(),
            None if lo_d is None else lo_d.data_ptr(), None if hi_d is None else hi_d.data_ptr(), max_rows, B,
            max_rows, max_cols, ti.data_ptr(), tj.data_ptr(), ln.data_ptr(), self._stream()))
        ti_h, tj_h, ln_h = ti.cpu().numpy(), tj.cpu().numpy(), ln.cpu().numpy()
        return [(ti_h[b, : ln_h[b]].astype(np.int64), tj_h[b, : ln_h[b]].astype(np.int64)) for b in range(B)]
