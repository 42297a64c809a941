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
