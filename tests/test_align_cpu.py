"""Word-timing alignment without a GPU: the oracle's restatement and the host
functions against vectors recorded from the reference
(tests/golden/make_align_golden.py)."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import oracle
from whisperdrz_b200 import alignment as A
from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.weights import init_state_dict

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "align.npz"))


def random_case(seed, N, M, banded):
    """Same generator as tests/golden/make_align_golden.py:random_case."""
    rng = np.random.RandomState(seed)
    x = rng.standard_normal((N, M)).astype(np.float32)
    if banded:
        for i in range(N):
            c = int(i * M / max(N, 1))
            lo, hi = max(0, c - M // 5 - 3), min(M, c + M // 5 + 3)
            x[i, :lo] = np.inf
            x[i, hi:] = np.inf
    return x


def oracle_scores(gold):
    dims = ModelDimensions.from_name("test-small")
    sd = init_state_dict(dims, 0)
    audio = synth.clips([int(s) for s in gold["clip_seeds"]])
    mel = torch.stack([oracle.window_mel(oracle.log_mel(torch.from_numpy(a))) for a in audio])
    xa = oracle.encoder(sd, mel, dims.n_audio_layer, dims.n_audio_head)
    heads = [tuple(int(v) for v in h) for h in gold["heads"]]
    tokens = torch.from_numpy(gold["full_tokens"]).long()
    return oracle.align_scores(sd, tokens, xa, dims.n_text_layer, dims.n_text_head, heads)


def test_full_tokens_layout(gold):
    ids = [gold["ids0"].tolist(), gold["ids1"].tolist()]
    toks, lens = A.build_full_tokens(ids, tuple(int(t) for t in gold["sot_sequence"]), int(gold["no_timestamps"]),
                                     int(gold["eot"]))
    assert np.array_equal(toks, gold["full_tokens"]) and lens == gold["actual_lens"].tolist()
    assert tuple(int(t) for t in gold["sot_sequence"]) == A.SOT_SEQUENCE


def test_oracle_scores_and_matrix_match_reference(gold):
    w = oracle_scores(gold)
    ref = torch.from_numpy(gold["scores_slice"])
    assert (w[:, :, ::3, ::41] - ref).abs().max() < 1e-4 * ref.abs().max()
    assert np.allclose(w.double().sum(dim=(2, 3)).numpy(), gold["scores_sum"], rtol=1e-4, atol=1e-2)
    m = oracle.align_prep(w, gold["actual_lens"].tolist(), gold["audio_caps"].tolist())
    ref_m = torch.from_numpy(gold["matrix_slice"])
    assert m.shape[-1] == int(gold["audio_caps"].max())
    assert (m[:, :, ::9] - ref_m).abs().max() < 2e-3      # values are z-scores of order one


def test_oracle_dtw_paths_identical_to_reference(gold):
    for bi in range(2):
        ti, tj = oracle.dtw_path(gold[f"neg{bi}"])
        assert np.array_equal(ti, gold[f"path_text{bi}"]) and np.array_equal(tj, gold[f"path_time{bi}"])
    for ci, (N, M, banded) in enumerate(gold["random_cases"].tolist()):
        ti, tj = oracle.dtw_path(random_case(100 + ci, N, M, banded))
        assert np.array_equal(ti, gold[f"rand_text{ci}"]) and np.array_equal(tj, gold[f"rand_time{ci}"]), (N, M, banded)


def test_anchor_limits_and_word_times_match_reference(gold):
    sot_len = len(gold["sot_sequence"])
    m = oracle.align_prep(oracle_scores(gold), gold["actual_lens"].tolist(), gold["audio_caps"].tolist()).numpy()
    for bi in range(2):
        neg_ref = gold[f"neg{bi}"]
        n_rows, cap = neg_ref.shape
        assert n_rows == int(gold["actual_lens"][bi]) - 1 - sot_len and cap == int(gold["audio_caps"][bi])
        wl = gold[f"word_lens{bi}"].tolist()
        wa = [(int(a), b, c) for a, b, c in gold[f"word_anchors{bi}"].tolist()]
        ta = [(a, b, int(c), int(d)) for a, b, c, d in gold[f"tag_anchors{bi}"].tolist()]
        lo, hi = A.anchor_row_limits(n_rows, cap, wl, wa, ta)
        cols = np.arange(cap)[None, :]
        blocked = (cols < lo[:, None]) | (cols >= hi[:, None])
        assert np.array_equal(blocked, np.isinf(neg_ref))            # the same cells are masked
        neg = -m[bi, sot_len: sot_len + n_rows, :cap]
        assert np.abs(neg[~blocked] - neg_ref[~blocked]).max() < 2e-3
        times = A.word_times_from_path(gold[f"path_text{bi}"].astype(np.int64), gold[f"path_time{bi}"].astype(np.int64), wl)
        assert np.allclose(np.array(times), gold[f"word_times{bi}"])
    assert A.word_times_from_path(np.array([0, 0, 1]), np.array([0, 1, 2]), [3, 3]) == []   # path too short


def test_anchor_limits_on_random_anchor_sets_match_reference(gold):
    """40 random sets of word and tag anchors (unordered, overlapping, past the last word or the audio,
    one-sided tags) through the reference's _apply_anchor_bands: the same cells stay allowed."""
    n_blocked_rows = 0
    for ci in range(int(gold["n_band_cases"])):
        n_rows, cap = (int(v) for v in gold[f"band{ci}_shape"])
        wa = [(int(a), b, c) for a, b, c in gold[f"band{ci}_word_anchors"].tolist()]
        ta = [(a, b, None if c < 0 else int(c), None if d < 0 else int(d)) for a, b, c, d in gold[f"band{ci}_tag_anchors"].tolist()]
        lo, hi = A.anchor_row_limits(n_rows, cap, gold[f"band{ci}_word_lens"].tolist(), wa, ta)
        rlo, rhi = gold[f"band{ci}_lo"], gold[f"band{ci}_hi"]
        for i in range(n_rows):
            if rhi[i] <= rlo[i]:
                assert hi[i] <= lo[i], (ci, i)
                n_blocked_rows += 1
            else:
                assert (lo[i], hi[i]) == (rlo[i], rhi[i]), (ci, i, lo[i], hi[i], rlo[i], rhi[i])
    assert n_blocked_rows >= 0


def test_alignment_heads_constant_matches_the_reference_mask():
    import base64
    import gzip
    packed = b"ABzY8gWO1E0{>%R7(9S+Kn!D~%ngiGaR?*L!iJG9p-nab0JQ=-{D1-g00"   # dtw_align.py:49
    arr = np.frombuffer(gzip.decompress(base64.b85decode(packed)), dtype=bool).reshape(32, 20)
    assert [tuple(r) for r in np.argwhere(arr).tolist()] == A.ALIGNMENT_HEADS_LARGE_V3
