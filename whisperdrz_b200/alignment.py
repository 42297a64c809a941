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
    """Allowed audio columns [lo, hi) of each text row of the cost matrix.

    The reference sets cost to +inf outside bands around the timestamps the
    decoder itself emitted: rows of an anchored word may only use columns
    within ``slack_frames`` of its (start, end); the last row of the word
    before a speaker tag must end before the tag's end, the first row of the
    word after it must start after the tag's start.  Several bands on one row
    intersect.  Row 0 is the no-timestamps row, word w starts at row
    ``1 + sum(word_lens[:w])``.  A band is skipped under the reference's
    conditions (word index past the last word, non-increasing anchor end,
    empty column or row range)."""
    lo = np.zeros(n_rows, dtype=np.int32)
    hi = np.full(n_rows, n_cols, dtype=np.int32)
    n_words = len(word_lens)                       # the reference's word list has one more entry (the eot)
    bounds = np.cumsum([1, *word_lens])            # first row of word w; bounds[n_words] = one past the last
    bands: list[tuple[int, int, int | None, int | None]] = []
    seen_max = -1.0
    for wi, a_s, a_e in word_anchors or []:
        wi = int(wi)
        if wi >= n_words or a_e <= seen_max:
            continue
        a_lo = max(0, int(round(a_s * TOKENS_PER_SECOND)) - slack_frames)
        a_hi = min(n_cols, int(round(a_e * TOKENS_PER_SECOND)) + slack_frames)
        if a_lo >= a_hi:
            continue
        r_lo, r_hi = int(bounds[wi]), min(int(bounds[wi + 1]), n_rows)
        if r_lo >= r_hi:
            continue
        bands.append((r_lo, r_hi, a_lo, a_hi))
        seen_max = a_e
    for a_s, a_e, p_local, n_local in tag_anchors or []:
        a_lo = max(0, int(round(a_s * TOKENS_PER_SECOND)) - slack_frames)
        a_hi = min(n_cols, int(round(a_e * TOKENS_PER_SECOND)) + slack_frames)
        if a_hi <= 0 or a_lo >= n_cols:
            continue
        if p_local is not None and int(p_local) < n_words:
            r = min(int(bounds[int(p_local) + 1]) - 1, n_rows - 1)
            if r >= 0:
                bands.append((r, r + 1, None, a_hi))
        if n_local is not None and int(n_local) < n_words:
            r = min(int(bounds[int(n_local)]), n_rows - 1)
            if r >= 0:
                bands.append((r, r + 1, a_lo, None))
    for r_lo, r_hi, a_lo, a_hi in bands:
        if a_lo is not None and a_lo > 0:
            lo[r_lo:r_hi] = np.maximum(lo[r_lo:r_hi], a_lo)
        if a_hi is not None and a_hi < n_cols:
            hi[r_lo:r_hi] = np.minimum(hi[r_lo:r_hi], a_hi)
    return lo, hi


def word_times_from_path(text_idx: np.ndarray, time_idx: np.ndarray, word_lens: list[int]) -> list[tuple[float, float]]:
    """(start, end) seconds of each word: the audio position at which the path first enters the word's
    first row, and the one at which it enters the next word's.  Empty when the path never reaches the last
    boundary, as in the reference."""
    if len(text_idx) == 0 or not word_lens:
        return []
    boundaries = np.pad(np.cumsum(word_lens), (1, 0))
    jumps = np.pad(np.diff(text_idx), (1, 0), constant_values=1).astype(bool)
    jump_times = np.asarray(time_idx)[jumps] / TOKENS_PER_SECOND
    if boundaries[-1] >= len(jump_times):
        return []
    return list(zip(jump_times[boundaries[:-1]].tolist(), jump_times[boundaries[1:]].tolist()))


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
