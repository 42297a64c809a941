"""CPU oracle for the transcription hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 torch on the CPU, the arithmetic of the
reference's log-mel front end, encoder, cached decoder and logit rules.  It is
the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  Nothing in the
``whisperdrz_b200`` package imports it; the product path runs only through the
CUDA library and fails if that library is missing.

Pinning: the reference ships no tests and no golden vectors for this path, so
the oracle is pinned against outputs of the reference itself, produced by
``tests/golden/make_golden.py`` (which imports the reference where it is
mounted) and committed under ``tests/golden/``.  ``tests/test_oracle_golden.py``
re-checks the oracle against those vectors on every CPU run.

Each function cites the reference lines it follows (paths inside the
reference project).  Third-party arithmetic the reference calls and that is
not in its tree (torch.stft, torchaudio ``melscale_fbanks`` with slaney
scale/norm, SDPA, LayerNorm, GELU; versions unpinned in pyproject.toml:12-23)
is restated from the published definitions.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

HEAD_DIM = 64
MASK_VALUE = -65504.0  # src/whisperdrz/decoding.py:1725-1728
REP_PENALTY = 1.2  # src/whisperdrz/decoding.py:1733


# --------------------------------------------------------------------------- #
# log-mel front end (src/whisperdrz/audio.py:81-156)
# --------------------------------------------------------------------------- #
def _hz_to_mel_slaney(f):
    f = np.asarray(f, dtype=np.float64)
    f_sp = 200.0 / 3
    mels = f / f_sp
    min_log_hz = 1000.0
    min_log_mel = min_log_hz / f_sp
    logstep = math.log(6.4) / 27.0
    with np.errstate(divide="ignore", invalid="ignore"):
        log_t = min_log_mel + np.log(np.maximum(f, 1e-300) / min_log_hz) / logstep
    return np.where(f >= min_log_hz, log_t, mels)


def _mel_to_hz_slaney(m):
    m = np.asarray(m, dtype=np.float64)
    f_sp = 200.0 / 3
    freqs = f_sp * m
    min_log_hz = 1000.0
    min_log_mel = min_log_hz / f_sp
    logstep = math.log(6.4) / 27.0
    return np.where(m >= min_log_mel, min_log_hz * np.exp(logstep * (m - min_log_mel)), freqs)


def mel_filterbank(n_freqs: int = 201, n_mels: int = 128, sample_rate: int = 16000,
                   f_min: float = 0.0, f_max: float | None = None) -> torch.Tensor:
    """Slaney-scale, slaney-normalised triangular filterbank ``[n_freqs, n_mels]``
    as built by torchaudio's ``MelScale`` (audio.py:98-104; f_max = sr/2)."""
    f_max = f_max if f_max is not None else sample_rate / 2.0
    all_freqs = torch.linspace(0, sample_rate // 2, n_freqs)
    m_pts = torch.linspace(float(_hz_to_mel_slaney(f_min)), float(_hz_to_mel_slaney(f_max)),
                           n_mels + 2)
    f_pts = torch.from_numpy(_mel_to_hz_slaney(m_pts.double().numpy())).to(torch.float32)
    f_diff = f_pts[1:] - f_pts[:-1]
    slopes = f_pts.unsqueeze(0) - all_freqs.unsqueeze(1)
    down = (-1.0 * slopes[:, :-2]) / f_diff[:-1]
    up = slopes[:, 2:] / f_diff[1:]
    fb = torch.clamp(torch.minimum(down, up), min=0.0)
    enorm = 2.0 / (f_pts[2: n_mels + 2] - f_pts[:n_mels])
    return fb * enorm.unsqueeze(0)


def log_mel(audio: torch.Tensor, n_mels: int = 128) -> torch.Tensor:
    """``LogMelSpectrogram._compute_mel_spec`` (audio.py:141-156): centred STFT
    with reflect padding, periodic Hann(400), hop 160; last frame dropped;
    power; mel; log10 clamp 1e-10; floor at (clip max - 8); (x + 4) / 4.
    audio fp32 [N] -> [n_mels, N // 160]."""
    x = audio.to(torch.float32)
    n_fft, hop = 400, 160
    xp = F.pad(x[None, None], (n_fft // 2, n_fft // 2), mode="reflect")[0, 0]
    frames = xp.unfold(0, n_fft, hop)  # [1 + N // hop, 400]
    win = torch.hann_window(n_fft, periodic=True, dtype=torch.float32)
    spec = torch.fft.rfft(frames * win, dim=-1)  # [T, 201]
    power = (spec.real ** 2 + spec.imag ** 2)[:-1]  # drop last frame
    fb = mel_filterbank(n_fft // 2 + 1, n_mels)
    mel = power @ fb  # [T, n_mels]
    log_spec = torch.clamp(mel, min=1e-10).log10()
    log_spec = torch.maximum(log_spec, log_spec.max() - 8.0)
    return ((log_spec + 4.0) / 4.0).T.contiguous()


def window_mel(mel: torch.Tensor, offset_frames: int = 0, target_frames: int = 3000) -> torch.Tensor:
    """Slice a chunk's mel at a window offset and pad with -1.5
    (src/whisperdrz/transcriber.py:1062-1072; audio.py:134-139)."""
    s = mel[:, offset_frames: offset_frames + target_frames]
    if s.shape[-1] < target_frames:
        s = F.pad(s, (0, target_frames - s.shape[-1]), value=-1.5)
    return s


# --------------------------------------------------------------------------- #
# transformer pieces (src/whisperdrz/model.py)
# --------------------------------------------------------------------------- #
def _ln(x, sd, p):
    # model.py:195-200, eps 1e-5 (nn.LayerNorm default)
    return F.layer_norm(x, (x.shape[-1],), sd[p + ".weight"], sd[p + ".bias"], 1e-5)


def _attend(q, k, v, mask=None):
    """softmax(q k^T / 8 + mask) v with q,k,v [B, T, H, 64] (model.py:69-75,288-296)."""
    q = q.permute(0, 2, 1, 3)
    k = k.permute(0, 2, 1, 3)
    v = v.permute(0, 2, 1, 3)
    s = (q @ k.transpose(-1, -2)) * (HEAD_DIM ** -0.5)
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    return (torch.softmax(s, dim=-1) @ v).permute(0, 2, 1, 3)


def _mlp(x, sd, p):
    # model.py:387-393, exact (erf) GELU
    h = F.gelu(F.linear(x, sd[p + ".mlp.0.weight"], sd[p + ".mlp.0.bias"]))
    return F.linear(h, sd[p + ".mlp.2.weight"], sd[p + ".mlp.2.bias"])


def encoder(sd: dict, mel: torch.Tensor, n_layer: int, n_head: int) -> torch.Tensor:
    """``AudioEncoder.forward`` (model.py:462-475). mel [B, n_mels, 3000] -> [B, 1500, d]."""
    x = F.gelu(F.conv1d(mel, sd["encoder.conv1.weight"], sd["encoder.conv1.bias"], padding=1))
    x = F.gelu(F.conv1d(x, sd["encoder.conv2.weight"], sd["encoder.conv2.bias"], stride=2, padding=1))
    x = x.permute(0, 2, 1)
    x = x + sd["encoder.positional_embedding"][: x.shape[1]]
    B, T, d = x.shape
    for i in range(n_layer):
        p = f"encoder.blocks.{i}"
        h = _ln(x, sd, p + ".attn_ln")
        q = F.linear(h, sd[p + ".attn.query.weight"], sd[p + ".attn.query.bias"])
        k = F.linear(h, sd[p + ".attn.key.weight"])
        v = F.linear(h, sd[p + ".attn.value.weight"], sd[p + ".attn.value.bias"])
        a = _attend(q.view(B, T, n_head, -1), k.view(B, T, n_head, -1), v.view(B, T, n_head, -1))
        x = x + F.linear(a.reshape(B, T, d), sd[p + ".attn.out.weight"], sd[p + ".attn.out.bias"])
        x = x + _mlp(_ln(x, sd, p + ".mlp_ln"), sd, p)
    return _ln(x, sd, "encoder.ln_post")


class SlotDecoder:
    """Cached decoder over slotted KV (model.py:98-193, 301-362, 404-434,
    570-617, 824-869) with the SDPA fallback semantics of model.py:20-76:
    new K/V are appended at the slot's current length, self-attention is
    causal over ``[0, pos]``, cross-attention reads all encoder positions."""

    def __init__(self, sd: dict, n_layer: int, n_head: int, n_slots: int,
                 max_tokens: int, n_audio_ctx: int = 1500):
        self.sd, self.L, self.H = sd, n_layer, n_head
        d = sd["decoder.ln.weight"].shape[0]
        self.d = d
        self.self_k = torch.zeros(n_layer, n_slots, max_tokens, n_head, HEAD_DIM)
        self.self_v = torch.zeros_like(self.self_k)
        self.cross_k = torch.zeros(n_layer, n_slots, n_audio_ctx, n_head, HEAD_DIM)
        self.cross_v = torch.zeros_like(self.cross_k)
        self.seq_lens = torch.zeros(n_slots, dtype=torch.int64)

    def set_cross(self, xa: torch.Tensor, slots) -> None:
        """model.py:852-855: K = key(xa) (no bias), V = value(xa)."""
        B, T, _ = xa.shape
        for l in range(self.L):
            p = f"decoder.blocks.{l}.cross_attn"
            k = F.linear(xa, self.sd[p + ".key.weight"]).view(B, T, self.H, HEAD_DIM)
            v = F.linear(xa, self.sd[p + ".value.weight"], self.sd[p + ".value.bias"]).view(B, T, self.H, HEAD_DIM)
            for i, s in enumerate(slots):
                self.cross_k[l, s, :T] = k[i]
                self.cross_v[l, s, :T] = v[i]

    def reset(self, slots) -> None:
        for s in slots:
            self.seq_lens[s] = 0

    def forward(self, tokens: torch.Tensor, slots, positions=None) -> torch.Tensor:
        """tokens int64 [B, S]; row b is appended to slot ``slots[b]`` starting
        at that slot's length (or ``positions[b]``).  Returns logits [B, S, V]."""
        sd = self.sd
        B, S = tokens.shape
        slots = [int(s) for s in slots]
        start = [int(self.seq_lens[s]) if positions is None else int(positions[i])
                 for i, s in enumerate(slots)]
        pos = torch.tensor([[st + t for t in range(S)] for st in start])
        x = sd["decoder.token_embedding.weight"][tokens] + sd["decoder.positional_embedding"][pos]
        for l in range(self.L):
            p = f"decoder.blocks.{l}"
            h = _ln(x, sd, p + ".attn_ln")
            q = F.linear(h, sd[p + ".attn.query.weight"], sd[p + ".attn.query.bias"]).view(B, S, self.H, HEAD_DIM)
            k = F.linear(h, sd[p + ".attn.key.weight"]).view(B, S, self.H, HEAD_DIM)
            v = F.linear(h, sd[p + ".attn.value.weight"], sd[p + ".attn.value.bias"]).view(B, S, self.H, HEAD_DIM)
            outs = []
            for i, s in enumerate(slots):
                st = start[i]
                self.self_k[l, s, st: st + S] = k[i]
                self.self_v[l, s, st: st + S] = v[i]
                kk = self.self_k[l, s, : st + S][None]
                vv = self.self_v[l, s, : st + S][None]
                jj = torch.arange(st + S)
                mask = jj[None, :] <= (st + torch.arange(S))[:, None]
                outs.append(_attend(q[i: i + 1], kk, vv, mask[None, None]))
            a = torch.cat(outs, 0).reshape(B, S, self.d)
            x = x + F.linear(a, sd[p + ".attn.out.weight"], sd[p + ".attn.out.bias"])
            h = _ln(x, sd, p + ".cross_attn_ln")
            q = F.linear(h, sd[p + ".cross_attn.query.weight"], sd[p + ".cross_attn.query.bias"]).view(B, S, self.H, HEAD_DIM)
            a = _attend(q, self.cross_k[l, slots], self.cross_v[l, slots]).reshape(B, S, self.d)
            x = x + F.linear(a, sd[p + ".cross_attn.out.weight"], sd[p + ".cross_attn.out.bias"])
            x = x + _mlp(_ln(x, sd, p + ".mlp_ln"), sd, p)
        for i, s in enumerate(slots):
            self.seq_lens[s] = start[i] + S
        x = _ln(x, sd, "decoder.ln")
        return x @ sd["decoder.token_embedding.weight"].T

    def prefill(self, tokens: torch.Tensor, xa: torch.Tensor, slots) -> torch.Tensor:
        """``WhisperDRZ.prefill_flash`` (model.py:824-869)."""
        self.set_cross(xa, slots)
        self.reset(slots)
        return self.forward(tokens, slots)


# --------------------------------------------------------------------------- #
# logit rules + greedy argmax (src/whisperdrz/decoding.py:1514-1777, 2033-2044)
# --------------------------------------------------------------------------- #
# A row's rule is a dict with the fields of ``wdz_rule_desc``:
#   forced_id, mode, arg0, arg1, table_bits, prefix_begin, prefix_end,
#   set_ids, clear_ids, pen_ids
MODE_OR, MODE_ALL_EXCEPT_TABLE, MODE_ALL_EXCEPT_RANGE, MODE_ALL = 0, 1, 2, 3


def blocked_mask(rule: dict, tables: torch.Tensor, V: int) -> torch.Tensor:
    """Boolean blocked-set of one row.  ``tables`` is bool [n_tables, V].
    Normal form of the ordered mask algebra of decoding.py:1527-1713: a base
    (nothing / everything except a table / everything except an id range /
    everything), OR-ed class tables (the first 32 by bit, one more by index),
    the complement of an allow-list table, a blocked id prefix range, single
    ids set, then single ids cleared."""
    mode = rule.get("mode", MODE_OR)
    if mode == MODE_OR:
        m = torch.zeros(V, dtype=torch.bool)
    elif mode == MODE_ALL_EXCEPT_TABLE:
        m = ~tables[rule["arg0"]].clone()
    elif mode == MODE_ALL_EXCEPT_RANGE:
        m = torch.ones(V, dtype=torch.bool)
        m[max(rule["arg0"], 0): max(min(rule["arg1"], V), 0)] = False
    else:
        m = torch.ones(V, dtype=torch.bool)
    bits = rule.get("table_bits", 0)
    for i in range(min(32, tables.shape[0])):
        if bits >> i & 1:
            m |= tables[i]
    if rule.get("or_table", 0) > 0:
        m |= tables[rule["or_table"]]
    if rule.get("allow_table", 0) > 0:
        m |= ~tables[rule["allow_table"]]
    pb, pe = rule.get("prefix_begin", 0), rule.get("prefix_end", 0)
    if pe > pb:
        m[max(pb, 0): min(pe, V)] = True
    for t in rule.get("set_ids", []):
        m[t] = True
    for t in rule.get("clear_ids", []):
        m[t] = False
    return m


def rules_argmax(logits: torch.Tensor, rules: list[dict], tables: torch.Tensor,
                 penalty: bool = True) -> torch.Tensor:
    """Phase 3 of ``decode_batch`` (decoding.py:1724-1762): additive -65504 on
    blocked ids, repetition penalty (/1.2 if > 0 else *1.2) on ``pen_ids``,
    argmax with the lowest index winning ties.  ``penalty=False`` is the
    Phase-4 re-argmax on raw logits (decoding.py:2033-2044)."""
    B, V = logits.shape
    out = torch.zeros(B, dtype=torch.int64)
    for b, rule in enumerate(rules):
        if rule.get("forced_id", -1) >= 0:
            out[b] = rule["forced_id"]
            continue
        m = blocked_mask(rule, tables, V)
        add = torch.zeros(V, dtype=logits.dtype)
        add.masked_fill_(m, MASK_VALUE)
        val = logits[b] + add
        pen = [t for t in set(rule.get("pen_ids", [])) if 0 <= t < V]
        if penalty and pen:
            pm = torch.zeros(V, dtype=torch.bool)
            pm[pen] = True
            penalized = torch.where(val > 0, val / REP_PENALTY, val * REP_PENALTY)
            val = torch.where(pm, penalized, val)
        out[b] = int(torch.argmax(val))
    return out


# --------------------------------------------------------------------------- #
# word-timing alignment (src/whisperdrz/dtw_align.py: device steps of
# fill_word_timings_batch, 1112-1240)
# --------------------------------------------------------------------------- #
def align_scores(sd: dict, tokens: torch.Tensor, xa: torch.Tensor, n_layer: int, n_head: int,
                 heads: list[tuple[int, int]]) -> torch.Tensor:
    """Teacher-forced uncached decoder pass (``TextDecoder.forward`` model.py:547-568 without the optional
    timing embedding, blocks as model.py:396-401) capturing, per decoder block, the cross-attention query
    and key projections (``CrossAttnCapture`` dtw_align.py:498-551), then ``compute_attention``
    (dtw_align.py:553-586): QK^T of the selected (layer, head) pairs with the hd^-0.25 scale on each side,
    no softmax.  tokens int64 [B, T], xa [B, Ta, d] -> f32 [B, n_sel, T, Ta].  Layers after the last
    selected one cannot change the result and are not run."""
    B, T = tokens.shape
    d = sd["decoder.ln.weight"].shape[0]
    x = sd["decoder.token_embedding.weight"][tokens] + sd["decoder.positional_embedding"][:T]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))[None, None]
    last = max(l for l, _ in heads)
    cap_q, cap_k = {}, {}
    for l in range(min(n_layer, last + 1)):
        p = f"decoder.blocks.{l}"
        h = _ln(x, sd, p + ".attn_ln")
        q = F.linear(h, sd[p + ".attn.query.weight"], sd[p + ".attn.query.bias"]).view(B, T, n_head, HEAD_DIM)
        k = F.linear(h, sd[p + ".attn.key.weight"]).view(B, T, n_head, HEAD_DIM)
        v = F.linear(h, sd[p + ".attn.value.weight"], sd[p + ".attn.value.bias"]).view(B, T, n_head, HEAD_DIM)
        x = x + F.linear(_attend(q, k, v, causal).reshape(B, T, d), sd[p + ".attn.out.weight"], sd[p + ".attn.out.bias"])
        h = _ln(x, sd, p + ".cross_attn_ln")
        q = F.linear(h, sd[p + ".cross_attn.query.weight"], sd[p + ".cross_attn.query.bias"])
        k = F.linear(xa, sd[p + ".cross_attn.key.weight"])
        v = F.linear(xa, sd[p + ".cross_attn.value.weight"], sd[p + ".cross_attn.value.bias"])
        cap_q[l], cap_k[l] = q, k
        Ta = xa.shape[1]
        a = _attend(q.view(B, T, n_head, HEAD_DIM), k.view(B, Ta, n_head, HEAD_DIM), v.view(B, Ta, n_head, HEAD_DIM))
        x = x + F.linear(a.reshape(B, T, d), sd[p + ".cross_attn.out.weight"], sd[p + ".cross_attn.out.bias"])
        x = x + _mlp(_ln(x, sd, p + ".mlp_ln"), sd, p)
    scale = HEAD_DIM ** -0.25
    out = []
    for l, hd in heads:
        qh = cap_q[l].view(B, T, n_head, HEAD_DIM)[:, :, hd].float() * scale
        kh = cap_k[l].view(B, -1, n_head, HEAD_DIM)[:, :, hd].float() * scale
        out.append(qh @ kh.transpose(-1, -2))
    return torch.stack(out, 1)


def median_filter7(x: torch.Tensor, width: int = 7) -> torch.Tensor:
    """Median along the last dim with reflect padding (dtw_align.py:65-84)."""
    pad = width // 2
    if x.shape[-1] <= pad:
        return x
    flat = F.pad(x.reshape(-1, 1, x.shape[-1]), (pad, pad), mode="reflect")
    return flat.unfold(-1, width, 1).sort(dim=-1).values[..., width // 2].reshape(x.shape)


def align_prep(weights: torch.Tensor, actual_lens: list[int], audio_caps: list[int], medfilt_width: int = 7) -> torch.Tensor:
    """``_dtw_prep_batch`` (dtw_align.py:700-753): columns at or past a chunk's audio cap are masked out of
    the softmax, mean / variance over the chunk's valid text rows per (head, audio column), normalise with
    std = sqrt(max(var, 1e-12)), median filter along audio over the full width, mean over heads.
    weights f32 [B, H, T, Ta] -> f32 [B, T, max(audio_caps)]."""
    B, H, T, Ta = weights.shape
    lens = torch.tensor(actual_lens)
    caps = torch.tensor(audio_caps)
    audio_mask = torch.arange(Ta)[None, :] < caps[:, None]
    w = weights.masked_fill(~audio_mask[:, None, None, :], float("-inf"))
    w = torch.softmax(w, dim=-1)
    tm = (torch.arange(T)[None, :] < lens[:, None])[:, None, :, None].to(w.dtype)
    n = lens.view(B, 1, 1, 1).to(w.dtype)
    mean = (w * tm).sum(dim=-2, keepdim=True) / n
    var = (((w - mean) ** 2) * tm).sum(dim=-2, keepdim=True) / n
    w = (w - mean) / var.clamp_min(1e-12).sqrt()
    if medfilt_width > 1:
        w = median_filter7(w, medfilt_width)
    return w.mean(dim=1)[:, :, : int(caps.max())].contiguous()


def dtw_path(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """``_dtw_numba`` (dtw_align.py:170-223): cost[i, j] = x[i-1, j-1] + min(diagonal, up, left) in float32
    with ties resolved diagonal, then up (text index), then left (time index); backtrace from (N, M) with
    the borders forcing 'left' on row 0 and 'up' on column 0.  Evaluated one anti-diagonal at a time.
    Returns (text_idx, time_idx) int64, both of the path length."""
    x = np.asarray(x, dtype=np.float32)
    N, M = x.shape
    cost = np.full((N + 1, M + 1), np.inf, dtype=np.float32)
    trace = np.full((N + 1, M + 1), -1, dtype=np.int8)
    trace[0, :] = 2
    trace[:, 0] = 1
    trace[0, 0] = -1
    cost[0, 0] = 0.0
    for k in range(2, N + M + 1):
        i = np.arange(max(1, k - M), min(N, k - 1) + 1)
        j = k - i
        c0, c1, c2 = cost[i - 1, j - 1], cost[i - 1, j], cost[i, j - 1]
        t = np.where((c0 <= c1) & (c0 <= c2), 0, np.where(c1 <= c2, 1, 2)).astype(np.int8)
        c = np.where(t == 0, c0, np.where(t == 1, c1, c2))
        cost[i, j] = x[i - 1, j - 1] + c
        trace[i, j] = t
    i, j = N, M
    ti, tj = [], []
    while i > 0 or j > 0:
        ti.append(i - 1)
        tj.append(j - 1)
        t = trace[i, j]
        if t == 0:
            i, j = i - 1, j - 1
        elif t == 1:
            i -= 1
        else:
            j -= 1
    return np.array(ti[::-1], dtype=np.int64), np.array(tj[::-1], dtype=np.int64)
