"""Word-timing alignment on the GPU through the C ABI: cost matrix against the
oracle, DTW paths bit-exact against paths recorded from the reference."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from whisperdrz_b200 import alignment as A
from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.weights import init_state_dict

from test_align_cpu import random_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "align.npz"))


def _engine(dtype, max_rows=None):
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name("test-small")
    sd = init_state_dict(dims, 0)
    return Engine(dims, sd, dtype=dtype, n_slots=4, max_clips=2, max_rows=max_rows), dims, sd


def _setup(e, gold, slots):
    audio = synth.clips([int(s) for s in gold["clip_seeds"]])
    xa = e.encode(e.logmel(torch.from_numpy(audio).cuda()))
    e.cross_kv(xa, slots)
    e.align_configure(gold["heads"])
    return xa


@pytest.mark.parametrize("dtype,max_rows,tol", [(torch.float32, None, 2e-3), (torch.float32, 16, 2e-3),
                                                (torch.bfloat16, None, 0.25)])
def test_align_matrix_matches_oracle_and_reference(gold, dtype, max_rows, tol):
    """fp32: the matrix (z-scores of order one) within 2e-3 of the reference's recorded slices and of the
    oracle on the engine's own encoder output; 16-row passes (the chunk is split across several forward
    calls) give the same.  bf16: a looser bound, and the path still follows the oracle's closely."""
    e, dims, sd = _engine(dtype, max_rows)
    slots = [2, 0]
    _setup(e, gold, slots)
    lens, caps = gold["actual_lens"].tolist(), gold["audio_caps"].tolist()
    m = e.align_matrix(gold["full_tokens"], lens, slots, caps).cpu()
    e.device_status()
    ref = torch.from_numpy(gold["matrix_slice"])
    T = ref.shape[1]
    for b in range(2):
        got = m[b, : lens[b], : max(caps)][:, ::9]
        assert (got - ref[b, : lens[b]]).abs().max() < tol, (b, float((got - ref[b, : lens[b]]).abs().max()))
        assert float(m[b, lens[b]:].abs().max() if lens[b] < T else 0.0) == 0.0     # padding rows are zero
        assert float(m[b, :, caps[b]:].abs().max() if caps[b] < dims.n_audio_ctx else 0.0) < 1e-3 + tol
    e.close()


def test_dtw_paths_identical_to_reference(gold):
    e, dims, _ = _engine(torch.float32)
    # the reference's own matrices (already negated and band-masked): feed -neg with the bands as limits
    for bi in range(2):
        neg = gold[f"neg{bi}"]
        n_rows, cap = neg.shape
        blocked = np.isinf(neg)
        lo = np.array([int(np.argmax(~blocked[i])) for i in range(n_rows)], dtype=np.int32)
        hi = np.array([cap - int(np.argmax(~blocked[i][::-1])) for i in range(n_rows)], dtype=np.int32)
        mat = torch.from_numpy(np.where(blocked, 0.0, -neg).astype(np.float32))
        (ti, tj), = e.dtw(mat, [0], [n_rows], [cap], [(lo, hi)])
        assert np.array_equal(ti, gold[f"path_text{bi}"]) and np.array_equal(tj, gold[f"path_time{bi}"])
    # seeded matrices of many shapes, several per launch, with row offsets and ragged sizes
    cases = gold["random_cases"].tolist()
    mats, limits = [], []
    for ci, (N, M, banded) in enumerate(cases):
        x = random_case(100 + ci, N, M, banded)
        blocked = np.isinf(x)
        lo = np.array([int(np.argmax(~blocked[i])) for i in range(N)], dtype=np.int32)
        hi = np.array([M - int(np.argmax(~blocked[i][::-1])) for i in range(N)], dtype=np.int32)
        mats.append(np.where(blocked, 0.0, -x).astype(np.float32))
        limits.append((lo, hi))
    row0 = [3 if N < 400 else 0 for N, _, _ in cases]
    big = np.zeros((len(cases), 448, 1500), dtype=np.float32)
    for ci, (N, M, _) in enumerate(cases):
        big[ci, row0[ci]: row0[ci] + N, :M] = mats[ci]
    paths = e.dtw(torch.from_numpy(big), row0, [c[0] for c in cases], [c[1] for c in cases], limits)
    e.device_status()
    for ci, (ti, tj) in enumerate(paths):
        assert np.array_equal(ti, gold[f"rand_text{ci}"]) and np.array_equal(tj, gold[f"rand_time{ci}"]), cases[ci]
    assert e.dtw(torch.zeros(1, 4, 4), [0], [0], [4])[0][0].size == 0         # empty chunk: empty path
    with pytest.raises(Exception):
        e.dtw(torch.zeros(1, 600, 8), [0], [600], [8])                          # more rows than one CTA takes
    e.close()


def test_align_chunks_end_to_end_word_times(gold):
    """alignment.align_chunks on the engine: fp32 word times equal the reference's (same path), with the
    anchors of chunk 1; a second chunk in the same slot is run in a second call."""
    e, dims, _ = _engine(torch.float32)
    slots = [1, 3]
    _setup(e, gold, slots)
    chunks = []
    for bi in range(2):
        wa = [(int(a), b, c) for a, b, c in gold[f"word_anchors{bi}"].tolist()]
        ta = [(a, b, int(c), int(d)) for a, b, c, d in gold[f"tag_anchors{bi}"].tolist()]
        chunks.append(A.AlignChunk(slot=slots[bi], ids=gold[f"ids{bi}"].tolist(), word_lens=gold[f"word_lens{bi}"].tolist(),
                                   num_frames=2 * int(gold["audio_caps"][bi]), word_anchors=wa, tag_anchors=ta))
    chunks.append(chunks[0])                                   # same slot again -> its own call
    times = A.align_chunks(e, chunks)
    e.device_status()
    for bi in range(2):
        assert np.allclose(np.array(times[bi]), gold[f"word_times{bi}"], atol=0.0201), (times[bi], gold[f"word_times{bi}"])
    assert times[2] == times[0]
    e.close()


def test_tensor_core_pass_matches_row_wise_pass_on_long_chunks(gold):
    """bf16, chunks of 300 and 170 tokens: with room for whole chunks in one forward call the pass runs its
    attention on tcgen05 (several 128-query tiles, causal diagonal tiles, ragged lengths); with max_rows
    below the chunk length it falls back to the row-wise decode kernels.  Same matrices up to bf16 noise,
    and both close to the fp32 oracle."""
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name("test-small")
    sd = init_state_dict(dims, 0)
    rng = np.random.RandomState(11)
    ids = [rng.randint(0, 50000, size=295).tolist(), rng.randint(0, 50000, size=165).tolist()]
    tokens, lens = A.build_full_tokens(ids)
    caps = [1500, 1100]
    slots = [1, 2]
    out = []
    xa_keep = None
    for max_rows in (320, 64):
        e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=4, max_clips=2, max_rows=max_rows)
        xa_keep = _setup(e, gold, slots)
        out.append(e.align_matrix(tokens, lens, slots, caps).cpu())
        e.device_status()
        e.close()
    for b in range(2):
        a, c = out[0][b, : lens[b]], out[1][b, : lens[b]]
        assert (a - c).abs().max() < 0.15 and (a - c).abs().mean() < 0.01, (float((a - c).abs().max()), float((a - c).abs().mean()))
    heads = [tuple(int(v) for v in h) for h in gold["heads"]]
    w = oracle.align_scores(sd, torch.from_numpy(tokens).long(), xa_keep.float().cpu(), dims.n_text_layer, dims.n_text_head, heads)
    m = oracle.align_prep(w, lens, caps)
    for b in range(2):
        diff = (out[0][b, : lens[b], : max(caps)] - m[b, : lens[b]]).abs()
        assert diff.mean() < 0.02 and diff.max() < 0.5, (float(diff.mean()), float(diff.max()))


def test_load_model_with_word_timing_end_to_end():
    """load_model(dtw_align=True): every finished window is aligned on the engine before its slot is reused;
    chunks carry one (token index, start, end) per text token, inside the chunk's time range, and the token
    ids are the same as without alignment (the pass must not disturb decoding)."""
    import whisperdrz_b200
    from whisperdrz_b200.dims import TOK_EOT
    audio = torch.from_numpy(synth.long_form(3, 70.0))
    out = {}
    for align in (False, True):
        t = whisperdrz_b200.load_model("test-small", n_slots=2, max_clips=2, dtype=torch.float32, max_new_tokens=40,
                                       dtw_align=align, align_heads=[(0, 1), (1, 0), (1, 3)])
        out[align] = t.transcribe(audio)
        t.engine.device_status()
        if align:
            assert t.windows_aligned >= len(out[align].raw_chunks) == 3
        t.engine.close()
    for a, b in zip(out[False].raw_chunks, out[True].raw_chunks):
        assert a["tokens"] == b["tokens"] and a["stop_reason"] == b["stop_reason"]
        words = b["word_times"]
        text_pos = [i for i, tk in enumerate(b["tokens"]) if tk < TOK_EOT]
        assert sorted(w[0] for w in words) == [w[0] for w in words] and set(w[0] for w in words) <= set(text_pos)
        assert len(words) >= 1
        assert all(b["offset"] - 1e-6 <= w[1] <= w[2] <= b["offset"] + 30.0 + 1e-6 for w in words)
