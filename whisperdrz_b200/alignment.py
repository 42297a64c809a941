"""Word-timing alignment: host side of the device steps of the reference's
``fill_word_timings_batch`` (src/whisperdrz/dtw_align.py:1112-1303).

The reference fills in word timings after a window has been decoded: it
re-tokenises the predicted text at character level, runs the decoder once over
those tokens with hooks on the cross-attention projections of the alignment
heads, turns their QK^T into a cost matrix (softmax, normalise, median filter,
head mean) and finds the monotonic text-to-audio path by dynamic time warping.
Text parsing and re-rendering stay host string code on the caller's side; this
module covers everything from token ids to word times:

* ``build_full_tokens``  - sot sequence + no-timestamps + ids + eot, eot-padded
  (``_build_full_tokens_batch`` dtw_align.py:1096-1109);
* ``Engine.align_matrix`` - teacher-forced pass against the slot's cached cross
  keys, scores of the alignment heads and the fused preparation
  (``CrossAttnCapture`` :498-586 and ``_dtw_prep_batch`` :700-753);
* ``anchor_row_limits``  - the anchor bands of ``_apply_anchor_bands``
  (:589-641) as an allowed column range per text row;
* ``Engine.dtw``         - cost accumulation and backtrace (``_dtw_numba`` :170-223);
* ``word_times_from_path`` - path to per-word (start, end) seconds
  (``_dtw_from_neg_matrix`` :644-667).

``align_chunks`` strings them together for a batch of chunks.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .dims import TOK_EOT, TOK_LANG_EN, TOK_NO_TIMESTAMPS, TOK_SOT, TOK_TRANSCRIBE

TOKENS_PER_SECOND = 50.0   # audio positions of the encoder per second (src/whisperdrz/audio.py:22-24)
FRAMES_PER_SECOND = 100

# (layer, head) pairs whose cross-attention tracks time in large-v3; the reference stores them as a
# compressed bitmask (dtw_align.py:49) that decodes to this list.
ALIGNMENT_HEADS_LARGE_V3 = [(7, 0), (10, 17), (12, 18), (13, 12), (16, 1), (17, 14), (19, 11), (21, 4), (24, 1), (25, 6)]

SOT_SEQUENCE = (TOK_SOT, TOK_LANG_EN, TOK_TRANSCRIBE)


@dataclass
class AlignChunk:
    """One chunk of predicted text to align against the audio window cached in ``slot``."""
    slot: int
    ids: list[int]                       # character-level token ids of the rendered text
    word_lens: list[int]                 # tokens per word, in order (sum = len(ids))
    num_frames: int = 3000               # mel frames of real audio in the window
    word_anchors: list[tuple[int, float, float]] = field(default_factory=list)
    tag_anchors: list[tuple[float, float, int | None, int | None]] = field(default_factory=list)


def build_full_tokens(ids_list: list[list[int]], sot_sequence=SOT_SEQUENCE, no_timestamps: int = TOK_NO_TIMESTAMPS,
                      eot: int = TOK_EOT) -> tuple[np.ndarray, list[int]]:
    """Right-pads each chunk's sot + no_timestamps + ids + eot with eot.  Returns (int32 [B, T], lengths)."""
    sot = list(sot_sequence)
    lens = [len(sot) + 1 + len(ids) + 1 for ids in ids_list]
    out = np.full((len(ids_list), max(lens)), eot, dtype=np.int32)
    for b, ids in enumerate(ids_list):
        seq = [*sot, no_timestamps, *ids, eot]
        out[b, : len(seq)] = seq
    return out, lens


def anchor_row_limits(n_rows: int, n_cols: int, word_lens: list[int],
                      word_anchors=None, tag_anchors=None, slack_frames: int = 7) -> tuple[np.ndarray, np.ndarray]:
    """Allowed audio columns [lo, hi) of each text row of the cost matrix, as two int32 arrays.

    Where the decoder itself emitted timestamps, the reference forbids (cost +inf) everything outside
    bands around them (dtw_align.py:589-641); the device DTW takes the same constraint as a column
    interval per row, so nothing is written into the matrix.  Rows: row 0 is the no-timestamps token,
    word w owns rows ``first[w] .. first[w + 1] - 1`` with ``first = 1 + exclusive cumsum(word_lens)``.

    * a timed word (index, start, end) keeps its rows within ``slack_frames`` positions of
      [start, end].  Anchors are honoured in list order only while their end times strictly increase;
      an anchor is also void when its word index, its column span or its row span is empty.
    * a timed tag (start, end, previous word, next word) makes the last row of the previous word end
      before the tag's end and the first row of the next word start after the tag's start.
    Several constraints on one row intersect."""
    lo = np.zeros(n_rows, dtype=np.int32)
    hi = np.full(n_rows, n_cols, dtype=np.int32)
    n_words = len(word_lens)
    first = 1 + np.concatenate([[0], np.cumsum(word_lens)]).astype(np.int64)      # [n_words + 1]

    def col(t):   # seconds -> audio position
        return np.rint(np.asarray(t, dtype=np.float64) * TOKENS_PER_SECOND).astype(np.int64)

    wa = np.asarray(word_anchors if word_anchors is not None and len(word_anchors) else np.zeros((0, 3)), dtype=np.float64).reshape(-1, 3)
    if len(wa):
        w = wa[:, 0].astype(np.int64)
        c_lo = np.maximum(0, col(wa[:, 1]) - slack_frames)
        c_hi = np.minimum(n_cols, col(wa[:, 2]) + slack_frames)
        inside = w < n_words
        wc = np.where(inside, w, 0)
        r_lo, r_hi = first[wc], np.minimum(first[wc + 1], n_rows)
        usable = inside & (c_lo < c_hi) & (r_lo < r_hi)
        # "end times strictly increase": compare with the largest end among the usable anchors before it
        ends = np.where(usable, wa[:, 2], -np.inf)
        before = np.concatenate([[-1.0], np.maximum.accumulate(ends)[:-1]])
        keep = usable & (wa[:, 2] > np.maximum(before, -1.0))
        for k in np.nonzero(keep)[0]:
            rows = slice(int(r_lo[k]), int(r_hi[k]))
            if c_lo[k] > 0:
                lo[rows] = np.maximum(lo[rows], c_lo[k])
            if c_hi[k] < n_cols:
                hi[rows] = np.minimum(hi[rows], c_hi[k])
    for t_s, t_e, prev_w, next_w in tag_anchors or []:
        c_lo = max(0, int(col(t_s)) - slack_frames)
        c_hi = min(n_cols, int(col(t_e)) + slack_frames)
        if c_hi <= 0 or c_lo >= n_cols:
            continue
        if prev_w is not None and int(prev_w) < n_words and c_hi < n_cols:
            r = min(int(first[int(prev_w) + 1]) - 1, n_rows - 1)
            if r >= 0:
                hi[r] = min(hi[r], c_hi)
        if next_w is not None and int(next_w) < n_words and c_lo > 0:
            r = min(int(first[int(next_w)]), n_rows - 1)
            if r >= 0:
                lo[r] = max(lo[r], c_lo)
    return lo, hi


def word_times_from_path(text_idx: np.ndarray, time_idx: np.ndarray, word_lens: list[int]) -> list[tuple[float, float]]:
    """(start, end) seconds of each word from a DTW path (dtw_align.py:644-667).  The path visits the text
    rows in order without skipping any, so the moment it enters row r is ``time_idx`` at the first path
    step whose row is r; a word starts when the path enters its first row and ends when it enters the
    next word's first row.  Empty when the path stops before the row after the last word."""
    if len(text_idx) == 0 or not word_lens:
        return []
    edges = np.concatenate([[0], np.cumsum(word_lens)]).astype(np.int64)     # first row of each word, and one past
    text_idx = np.asarray(text_idx)
    if edges[-1] > int(text_idx[-1]) - int(text_idx[0]):
        return []
    entered = np.searchsorted(text_idx, text_idx[0] + edges, side="left")
    t = np.asarray(time_idx)[entered] / TOKENS_PER_SECOND
    return list(zip(t[:-1].tolist(), t[1:].tolist()))


def token_aligner(tokens: list[int], ts_begin: int = 50365, ts_end: int = 51865, eot: int = TOK_EOT, max_tokens: int = 440) -> list[dict]:
    """Chunk records for the generated tokens of one window when no tokenizer is at hand: every text token
    is a word of one token (timestamp and special tokens are dropped), and a timestamp pair that encloses
    exactly one text token anchors it, as the reference anchors a word the decoder timed itself.
    A caller that holds the tokenizer passes its own function instead, re-tokenising the text at character
    level as the reference does (``tokens_chars`` dtw_align.py:256-293).  Returns a list of dicts with
    ids, word_lens, word_anchors, tag_anchors and token_pos (index of each word's token in ``tokens``),
    split so that no chunk exceeds ``max_tokens`` ids."""
    ids, pos, anchors = [], [], []
    open_t, inside = None, []
    for i, t in enumerate(tokens):
        if ts_begin <= t <= ts_end:
            sec = (t - ts_begin) * 0.02
            if open_t is None:
                open_t, inside = sec, []
            else:
                if len(inside) == 1:
                    anchors.append((inside[0], open_t, sec))
                open_t = None
        elif t < eot:
            if open_t is not None:
                inside.append(len(ids))
            ids.append(int(t))
            pos.append(i)
    out = []
    for c0 in range(0, len(ids), max_tokens):
        c1 = min(len(ids), c0 + max_tokens)
        out.append({"ids": ids[c0:c1], "word_lens": [1] * (c1 - c0), "token_pos": pos[c0:c1], "tag_anchors": [],
                    "word_anchors": [(w - c0, a, b) for w, a, b in anchors if c0 <= w < c1]})
    return [c for c in out if c["ids"]]


def align_chunks(engine, chunks: list[AlignChunk], sot_sequence=SOT_SEQUENCE, no_timestamps: int = TOK_NO_TIMESTAMPS,
                 eot: int = TOK_EOT, slack_frames: int = 7) -> list[list[tuple[float, float]]]:
    """Word times of every chunk.  Chunks of one call must sit in distinct slots (a second chunk of the
    same window goes into the next call): the teacher-forced pass reuses the slot's self-attention rows,
    which are free once the window has been decoded, and reads its cross keys."""
    if not chunks:
        return []
    out: list[list[tuple[float, float]] | None] = [None] * len(chunks)
    pending = list(range(len(chunks)))
    while pending:
        batch, seen, rest = [], set(), []
        for i in pending:
            (rest if chunks[i].slot in seen else batch).append(i)
            seen.add(chunks[i].slot)
        pending = rest
        tokens, lens = build_full_tokens([chunks[i].ids for i in batch], sot_sequence, no_timestamps, eot)
        n_ctx = engine.dims.n_audio_ctx
        caps = [max(0, min(int(chunks[i].num_frames) // 2, n_ctx)) for i in batch]
        matrix = engine.align_matrix(tokens, lens, [chunks[i].slot for i in batch], caps)
        sot_len = len(sot_sequence)
        row0 = [sot_len] * len(batch)
        n_rows = [ln - 1 - sot_len for ln in lens]
        limits = [anchor_row_limits(n_rows[k], caps[k], chunks[i].word_lens, chunks[i].word_anchors,
                                    chunks[i].tag_anchors, slack_frames) for k, i in enumerate(batch)]
        paths = engine.dtw(matrix, row0, n_rows, caps, limits)
        for k, i in enumerate(batch):
            ti, tj = paths[k]
            out[i] = word_times_from_path(ti, tj, chunks[i].word_lens) if n_rows[k] > 0 and caps[k] > 0 else []
    return out
