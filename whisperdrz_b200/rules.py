"""Host half of the logit rules at token level: the timing-parity subset of the
reference's ``decode_batch`` (src/whisperdrz/decoding.py:971-2046).

The reference classifies each slot from its decoded *text* with regular
expressions and needs its tokenizer assets; what the device needs from that
classification is a compact per-row descriptor (``wdz_rule_desc``).  This
module produces those descriptors from token ids alone for the rules that do
not depend on text: timestamps come in open/close pairs, text only between
them, timestamps never move backwards (decoding.py:1682-1689), the first
timestamp lies in the first second (decoding.py:2090-2156), special tokens are
never sampled (inference_utils.py:76-174), EOT only between pairs
(decoding.py:1465-1475), the repetition penalty covers the last ten generated
tokens of text rows (decoding.py:1733-1759), and a row that reached its
length budget is forced to EOT on the host (decoding.py:1100-1107).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import capi
from .dims import TOK_EOT, TOK_TS_BEGIN, TOK_TS_END

T_SPECIAL, T_TIMINGS = 0, 1
BIT_SPECIAL, BIT_TIMINGS = 1 << T_SPECIAL, 1 << T_TIMINGS
N_TIMINGS = TOK_TS_END - TOK_TS_BEGIN + 1  # 1501
FIRST_TIMING_MAX = 50                      # <= 1.00 s
OPEN_AFTER_CLOSE_SPAN = 100                # next opening within 2 s of the last closing


def timestamp_tables(n_vocab: int) -> torch.Tensor:
    """bool [2, V]: table 0 = special tokens incl. EOT (50257..50364),
    table 1 = timestamp tokens (50365..51865)."""
    t = torch.zeros(2, n_vocab, dtype=torch.bool)
    t[T_SPECIAL, TOK_EOT:TOK_TS_BEGIN] = True
    t[T_TIMINGS, TOK_TS_BEGIN: TOK_TS_END + 1] = True
    return t


@dataclass
class RowState:
    """Per-slot decode state (the token-level part of InferenceState,
    inference_utils.py:217-302)."""
    max_new: int
    n_new: int = 0
    timing_count: int = 0
    last_timing: int = -1          # index of the last timestamp (0.02 s units)
    last_was_timing: bool = False
    recent: list = field(default_factory=list)
    done: bool = False
    tokens: list = field(default_factory=list)

    def rule(self) -> dict:
        if self.n_new >= self.max_new:
            return {"forced_id": TOK_EOT}
        if self.timing_count == 0:
            return {"mode": capi.MODE_ALL_EXCEPT_RANGE, "arg0": TOK_TS_BEGIN,
                    "arg1": TOK_TS_BEGIN + FIRST_TIMING_MAX + 1}
        open_pair = self.timing_count % 2 == 1
        if open_pair and self.last_was_timing:
            # a word must follow an opening timestamp
            return {"table_bits": BIT_SPECIAL | BIT_TIMINGS, "pen_ids": self.recent[-10:]}
        if open_pair:
            # more text, or a closing timestamp later than the opening one
            return {"table_bits": BIT_SPECIAL, "prefix_begin": TOK_TS_BEGIN,
                    "prefix_end": TOK_TS_BEGIN + self.last_timing + 1, "pen_ids": self.recent[-10:]}
        # between pairs: the next opening timestamp (not earlier than the last closing), or EOT
        lo = TOK_TS_BEGIN + self.last_timing
        hi = min(TOK_TS_END + 1, lo + OPEN_AFTER_CLOSE_SPAN)
        if self.last_timing >= N_TIMINGS - 1:
            return {"forced_id": TOK_EOT}
        return {"mode": capi.MODE_ALL_EXCEPT_RANGE, "arg0": lo, "arg1": hi, "clear_ids": [TOK_EOT]}

    def update(self, tok: int) -> None:
        """Bookkeeping of update_state_after_decode (decoding.py:878-963)."""
        self.tokens.append(tok)
        self.n_new += 1
        if tok == TOK_EOT or tok < 0:
            self.done = True
            return
        if TOK_TS_BEGIN <= tok <= TOK_TS_END:
            self.timing_count += 1
            self.last_timing = tok - TOK_TS_BEGIN
            self.last_was_timing = True
        else:
            self.last_was_timing = False
            self.recent.append(tok)
            if len(self.recent) > 10:
                del self.recent[0]


def segments(tokens: list[int], offset: float = 0.0) -> list[dict]:
    """Token ids -> [{start, end, tokens}] from the open/close timestamp pairs."""
    out, cur, start = [], [], None
    for t in tokens:
        if TOK_TS_BEGIN <= t <= TOK_TS_END:
            sec = (t - TOK_TS_BEGIN) * 0.02
            if start is None:
                start, cur = sec, []
            else:
                out.append({"start": round(start + offset, 2), "end": round(sec + offset, 2), "tokens": cur})
                start = None
        elif t != TOK_EOT and start is not None:
            cur.append(t)
    return out


class BatchRuleState:
    """The state of ``RowState`` for all slots at once, as numpy arrays, so that
    one decode step builds every active row's descriptor and absorbs every new
    token without a Python loop over rows (the reference spends its per-step
    host time in exactly such a loop, decoding.py:1098-1456)."""

    def __init__(self, n_slots: int, max_new: int):
        import numpy as np
        self.np = np
        self.max_new = np.full(n_slots, max_new, np.int64)
        self.n_new = np.zeros(n_slots, np.int64)
        self.timing_count = np.zeros(n_slots, np.int64)
        self.last_timing = np.full(n_slots, -1, np.int64)
        self.last_was_timing = np.zeros(n_slots, bool)
        self.recent = np.zeros((n_slots, 10), np.int32)
        self.n_recent = np.zeros(n_slots, np.int64)
        self.done = np.zeros(n_slots, bool)
        self.tokens = np.zeros((n_slots, max_new + 2), np.int32)

    def reset(self, slot: int, max_new: int | None = None) -> None:
        if max_new is not None:
            self.max_new[slot] = max_new
        self.n_new[slot] = self.timing_count[slot] = self.n_recent[slot] = 0
        self.last_timing[slot] = -1
        self.last_was_timing[slot] = self.done[slot] = False

    def rules_array(self, idx) -> "np.ndarray":
        """int32 [len(idx), 32] in ``wdz_rule_desc`` layout for the slots ``idx``."""
        np = self.np
        idx = np.asarray(idx, np.int64)
        n = len(idx)
        a = np.zeros((n, 32), np.int32)
        a[:, 0] = -1
        tc, last, lwt = self.timing_count[idx], self.last_timing[idx], self.last_was_timing[idx]
        forced = self.n_new[idx] >= self.max_new[idx]
        first = ~forced & (tc == 0)
        open_pair = ~forced & (tc % 2 == 1)
        after_open = open_pair & lwt
        in_text = open_pair & ~lwt
        between = ~forced & ~first & ~open_pair
        forced = forced | (between & (last >= N_TIMINGS - 1))
        between = between & ~forced
        a[forced, 0] = TOK_EOT
        a[first, 1] = capi.MODE_ALL_EXCEPT_RANGE
        a[first, 2] = TOK_TS_BEGIN
        a[first, 3] = TOK_TS_BEGIN + FIRST_TIMING_MAX + 1
        a[after_open, 4] = BIT_SPECIAL | BIT_TIMINGS
        a[in_text, 4] = BIT_SPECIAL
        a[in_text, 5] = TOK_TS_BEGIN
        a[in_text, 6] = (TOK_TS_BEGIN + last + 1)[in_text]
        lo = TOK_TS_BEGIN + last
        a[between, 1] = capi.MODE_ALL_EXCEPT_RANGE
        a[between, 2] = lo[between]
        a[between, 3] = np.minimum(TOK_TS_END + 1, lo + OPEN_AFTER_CLOSE_SPAN)[between]
        a[between, 16] = 1
        a[between, 17] = TOK_EOT
        pen = open_pair
        a[pen, 21] = self.n_recent[idx][pen]
        a[pen, 22:32] = self.recent[idx][pen]
        return a

    def update(self, idx, toks) -> "np.ndarray":
        """Absorbs one new token per slot in ``idx``; returns the done flags of those slots."""
        np = self.np
        idx = np.asarray(idx, np.int64)
        toks = np.asarray(toks, np.int64)
        self.tokens[idx, np.minimum(self.n_new[idx], self.tokens.shape[1] - 1)] = toks
        self.n_new[idx] += 1
        end = (toks == TOK_EOT) | (toks < 0)
        self.done[idx[end]] = True
        live = ~end
        is_t = live & (toks >= TOK_TS_BEGIN) & (toks <= TOK_TS_END)
        it = idx[is_t]
        self.timing_count[it] += 1
        self.last_timing[it] = toks[is_t] - TOK_TS_BEGIN
        self.last_was_timing[it] = True
        is_w = live & ~is_t
        iw = idx[is_w]
        self.last_was_timing[iw] = False
        full = self.n_recent[iw] >= 10
        if full.any():
            f = iw[full]
            self.recent[f, :9] = self.recent[f, 1:]
            self.recent[f, 9] = toks[is_w][full]
        nf = iw[~full]
        self.recent[nf, self.n_recent[nf]] = toks[is_w][~full]
        self.n_recent[nf] += 1
        return self.done[idx]

    def slot_tokens(self, slot: int) -> list[int]:
        return [int(t) for t in self.tokens[slot, : min(self.n_new[slot], self.tokens.shape[1])]]
