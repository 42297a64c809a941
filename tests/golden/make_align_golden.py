"""Record what the reference's word-timing alignment computes on the device side.

Run where the reference is mounted:

    PYTHONPATH=<reference>/src python tests/golden/make_align_golden.py [--large]

The unmodified reference runs on the CPU: ``CrossAttnCapture`` around
``model.decoder(full_tokens, xa)`` and ``compute_attention`` give the raw QK^T
of the chosen (layer, head) pairs, ``_dtw_prep_batch`` the cost matrices,
``_apply_anchor_bands`` the anchor masks, ``_dtw_numba`` the paths and
``_dtw_from_neg_matrix`` the word times.  ``_dtw_prep_batch`` ends with a
pinned-buffer copy and a device synchronise that exist only on CUDA; those two
calls are wrapped (a plain buffer, a no-op), the function itself is untouched.

Stored in align.npz: the inputs (clip seeds, char-level ids per chunk, heads,
audio caps, anchors), slices and sums of the raw scores, slices of the cost
matrices, the full negated and band-masked matrices the DTW ran on (a few
hundred KB), the paths and word times; and for seeded random matrices of
several shapes (up to 444 x 1500, some with blocked bands) the paths only;
and for 40 random sets of word / tag anchors the columns ``_apply_anchor_bands``
leaves open in every row.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from whisperdrz_b200 import synth  # noqa: E402
from whisperdrz_b200.dims import ModelDimensions  # noqa: E402
from whisperdrz_b200.weights import init_state_dict  # noqa: E402

import whisperdrz.dtw_align as D  # noqa: E402  (the reference)
from whisperdrz.audio import LogMelSpectrogram  # noqa: E402
from whisperdrz.config import Config, ModelDimensions as RefDims  # noqa: E402
from whisperdrz.model import WhisperDRZ  # noqa: E402

HEADS = [(0, 1), (1, 0), (1, 3)]
CLIP_SEEDS = [21, 22]
AUDIO_CAPS = [1500, 730]
WORD_LENS = [[4, 3, 5, 2, 7], [3, 3, 2, 4]]          # char-level tokens per word
# chunk 1 carries anchors: (word index, start s, end s) and (start s, end s, previous word, next word)
WORD_ANCHORS = [[], [(1, 3.2, 4.1)]]
TAG_ANCHORS = [[], [(9.0, 9.6, 2, 3)]]
RANDOM_CASES = [(1, 1, 0), (1, 9, 0), (7, 1, 0), (5, 9, 0), (60, 200, 0), (60, 200, 1), (444, 1500, 0), (444, 1500, 1),
                (101, 333, 1)]


def random_case(seed: int, N: int, M: int, banded: int) -> np.ndarray:
    """The seeded matrix of a DTW-only case; ``banded`` blocks everything outside a diagonal band."""
    rng = np.random.RandomState(seed)
    x = rng.standard_normal((N, M)).astype(np.float32)
    if banded:
        for i in range(N):
            c = int(i * M / max(N, 1))
            lo, hi = max(0, c - M // 5 - 3), min(M, c + M // 5 + 3)
            x[i, :lo] = np.inf
            x[i, hi:] = np.inf
    return x


def large():
    """Full-size case (``--large``): large-v3 dimensions, seeded weights, one 30 s clip, a 44-id chunk with two word
    anchors, the reference's own ten alignment heads.  Stores slices of the cost matrix, the DTW path of the
    band-masked matrix and the word times (align_large.npz, ~100 KB).  Needs ~14 GB of RAM and a few minutes."""
    dims = ModelDimensions.from_name("large-v3")
    m = WhisperDRZ(RefDims(**dims.as_dict()), config=Config()).float().eval()
    m.load_state_dict(init_state_dict(dims, 0), strict=False)
    tok = m.tokenizer
    tomel = LogMelSpectrogram(dims.n_mels)
    audio = synth.clips([1])
    mel = torch.stack([tomel(torch.from_numpy(a).unsqueeze(0), target_frames=3000)[0] for a in audio])
    with torch.inference_mode():
        xa = m.encoder(mel)
    word_lens = [5, 3, 6, 2, 7, 4, 4, 6, 3, 4]
    rng = np.random.RandomState(9)
    ids = [int(t) for t in rng.randint(0, 50000, size=sum(word_lens))]
    full_tokens, actual_lens = D._build_full_tokens_batch(tok, [ids], xa.device)
    head_mask = D.make_head_mask(m)
    heads = [tuple(r) for r in head_mask.nonzero().tolist()]
    with D.CrossAttnCapture(m, layers={l for l, _ in heads}) as cap:
        with torch.inference_mode():
            m.decoder(full_tokens, xa)
        weights = cap.compute_attention(head_mask)
    if weights.dim() == 3:
        weights = weights.unsqueeze(0)
    caps = [1380]
    orig_pin, orig_sync = D._pinned_host_buffer, torch.cuda.synchronize
    D._pinned_host_buffer = lambda shape, dtype: torch.empty(shape, dtype=dtype)
    torch.cuda.synchronize = lambda *a, **k: None
    try:
        matrices = D._dtw_prep_batch(weights, actual_lens, caps).copy()
    finally:
        D._pinned_host_buffer, torch.cuda.synchronize = orig_pin, orig_sync
    sot_len = len(tok.sot_sequence)
    words = [f"w{i}" for i in range(len(word_lens))] + [""]
    word_tokens, o = [], 0
    for n in word_lens:
        word_tokens.append(ids[o:o + n])
        o += n
    word_tokens.append([tok.eot])
    word_anchors = [(2, 6.4, 7.9), (7, 19.0, 20.5)]
    neg = np.ascontiguousarray(-matrices[0, sot_len: actual_lens[0] - 1, :caps[0]], dtype=np.float32)
    D._apply_anchor_bands(neg, words, word_tokens, caps[0], word_anchors, [], slack_frames=7)
    text_idx, time_idx = D._dtw_numba(neg)
    times = D._dtw_from_neg_matrix(neg, words, word_tokens)
    np.savez_compressed(
        os.path.join(HERE, "align_large.npz"), clip_seed=np.int64(1), heads=np.array(heads), ids=np.array(ids),
        word_lens=np.array(word_lens), audio_cap=np.int64(caps[0]), actual_len=np.int64(actual_lens[0]),
        word_anchors=np.array(word_anchors, dtype=np.float64), matrix_slice=matrices[0][:, ::7],
        xa_slice=xa[0, ::50].numpy(), path_text=text_idx.astype(np.int16), path_time=time_idx.astype(np.int16),
        word_times=np.array([[s, e] for _, s, e in times], dtype=np.float64))
    print("wrote align_large.npz", os.path.getsize(os.path.join(HERE, "align_large.npz")) // 1024, "KB; path", len(text_idx),
          "word times", [round(float(s), 2) for _, s, _ in times])


def main():
    if "--large" in sys.argv:
        return large()
    dims = ModelDimensions.from_name("test-small")
    m = WhisperDRZ(RefDims(**dims.as_dict()), config=Config()).float().eval()
    m.load_state_dict(init_state_dict(dims, 0), strict=False)
    tok = m.tokenizer
    tomel = LogMelSpectrogram(dims.n_mels)
    audio = synth.clips(CLIP_SEEDS)
    mel = torch.stack([tomel(torch.from_numpy(a).unsqueeze(0), target_frames=3000)[0] for a in audio])
    with torch.inference_mode():
        xa = m.encoder(mel)

    rng = np.random.RandomState(5)
    ids_list = [[int(t) for t in rng.randint(0, 50000, size=sum(w))] for w in WORD_LENS]
    full_tokens, actual_lens = D._build_full_tokens_batch(tok, ids_list, xa.device)
    head_mask = torch.zeros(dims.n_text_layer, dims.n_text_head, dtype=torch.bool)
    for l, h in HEADS:
        head_mask[l, h] = True
    with D.CrossAttnCapture(m, layers={l for l, _ in HEADS}) as cap:
        with torch.inference_mode():
            m.decoder(full_tokens, xa)
        weights = cap.compute_attention(head_mask)          # [B, n_sel, T_pad, 1500]
    assert [tuple(r) for r in head_mask.nonzero().tolist()] == HEADS

    orig_pin, orig_sync = D._pinned_host_buffer, torch.cuda.synchronize
    D._pinned_host_buffer = lambda shape, dtype: torch.empty(shape, dtype=dtype)
    torch.cuda.synchronize = lambda *a, **k: None
    try:
        matrices = D._dtw_prep_batch(weights, actual_lens, AUDIO_CAPS).copy()
    finally:
        D._pinned_host_buffer, torch.cuda.synchronize = orig_pin, orig_sync

    sot_len = len(tok.sot_sequence)
    out = {
        "clip_seeds": np.array(CLIP_SEEDS), "heads": np.array(HEADS), "audio_caps": np.array(AUDIO_CAPS),
        "sot_sequence": np.array(tok.sot_sequence), "no_timestamps": np.int64(tok.no_timestamps), "eot": np.int64(tok.eot),
        "full_tokens": full_tokens.numpy(), "actual_lens": np.array(actual_lens),
        "scores_slice": weights[:, :, ::3, ::41].numpy(), "scores_sum": weights.double().sum(dim=(2, 3)).numpy(),
        "matrix_slice": matrices[:, :, ::9],
    }
    for bi, ids in enumerate(ids_list):
        words = [f"w{i}" for i in range(len(WORD_LENS[bi]))] + [""]
        word_tokens, o = [], 0
        for n in WORD_LENS[bi]:
            word_tokens.append(ids[o:o + n])
            o += n
        word_tokens.append([tok.eot])
        cap_b = AUDIO_CAPS[bi]
        neg = np.ascontiguousarray(-matrices[bi, sot_len: actual_lens[bi] - 1, :cap_b], dtype=np.float32)
        if WORD_ANCHORS[bi] or TAG_ANCHORS[bi]:
            D._apply_anchor_bands(neg, words, word_tokens, cap_b, WORD_ANCHORS[bi], TAG_ANCHORS[bi], slack_frames=7)
        text_idx, time_idx = D._dtw_numba(neg)
        times = D._dtw_from_neg_matrix(neg, words, word_tokens)
        out[f"ids{bi}"] = np.array(ids)
        out[f"word_lens{bi}"] = np.array(WORD_LENS[bi])
        out[f"word_anchors{bi}"] = np.array(WORD_ANCHORS[bi], dtype=np.float64).reshape(-1, 3)
        out[f"tag_anchors{bi}"] = np.array(TAG_ANCHORS[bi], dtype=np.float64).reshape(-1, 4)
        out[f"neg{bi}"] = neg
        out[f"path_text{bi}"] = text_idx.astype(np.int16)
        out[f"path_time{bi}"] = time_idx.astype(np.int16)
        out[f"word_times{bi}"] = np.array([[s, e] for _, s, e in times], dtype=np.float64)
        print(f"chunk {bi}: {neg.shape} path {len(text_idx)} blocked {int(np.isinf(neg).sum())} words {len(times)}")
    # anchor bands alone: random word / tag anchors (unordered, overlapping, out of range, one-sided tags)
    # through _apply_anchor_bands on a zero matrix; stored as the allowed column range of every row
    arng = np.random.RandomState(17)
    n_band_cases = 40
    for ci in range(n_band_cases):
        n_words = int(arng.randint(1, 12))
        wl = [int(v) for v in arng.randint(1, 6, size=n_words)]
        n_rows = 1 + sum(wl) - int(arng.randint(0, 2))          # sometimes one row short of the last word
        cap_b = int(arng.choice([200, 730, 1500]))
        words = [f"w{i}" for i in range(n_words)] + [""]
        word_tokens = [[0] * n for n in wl] + [[tok.eot]]
        wa = []
        for _ in range(int(arng.randint(0, 5))):
            st = float(arng.uniform(-1.0, cap_b / 50.0 + 1.0))
            wa.append((int(arng.randint(0, n_words + 2)), round(st, 2), round(st + float(arng.uniform(-0.2, 3.0)), 2)))
        ta = []
        for _ in range(int(arng.randint(0, 3))):
            st = float(arng.uniform(-1.0, cap_b / 50.0 + 1.0))
            pl = None if arng.rand() < 0.3 else int(arng.randint(0, n_words + 1))
            nl = None if arng.rand() < 0.3 else int(arng.randint(0, n_words + 1))
            ta.append((round(st, 2), round(st + float(arng.uniform(0.0, 2.0)), 2), pl, nl))
        z = np.zeros((n_rows, cap_b), dtype=np.float32)
        D._apply_anchor_bands(z, words, word_tokens, cap_b, wa, ta, slack_frames=7)
        ok = ~np.isinf(z)
        lo = np.array([int(np.argmax(r)) if r.any() else 0 for r in ok], dtype=np.int32)
        hi = np.array([cap_b - int(np.argmax(r[::-1])) if r.any() else 0 for r in ok], dtype=np.int32)
        assert all(ok[i, lo[i]:hi[i]].all() and ok[i].sum() == hi[i] - lo[i] for i in range(n_rows))   # contiguous
        out[f"band{ci}_shape"] = np.array([n_rows, cap_b])
        out[f"band{ci}_word_lens"] = np.array(wl)
        out[f"band{ci}_word_anchors"] = np.array(wa, dtype=np.float64).reshape(-1, 3)
        out[f"band{ci}_tag_anchors"] = np.array([[a, b, -1 if c is None else c, -1 if d is None else d] for a, b, c, d in ta],
                                                dtype=np.float64).reshape(-1, 4)
        out[f"band{ci}_lo"], out[f"band{ci}_hi"] = lo, hi
    out["n_band_cases"] = np.int64(n_band_cases)
    out["random_cases"] = np.array(RANDOM_CASES)
    for ci, (N, M, banded) in enumerate(RANDOM_CASES):
        ti, tj = D._dtw_numba(random_case(100 + ci, N, M, banded))
        out[f"rand_text{ci}"] = ti.astype(np.int16)
        out[f"rand_time{ci}"] = tj.astype(np.int16)
    np.savez_compressed(os.path.join(HERE, "align.npz"), **out)
    print("wrote align.npz", os.path.getsize(os.path.join(HERE, "align.npz")) // 1024, "KB")


if __name__ == "__main__":
    main()
