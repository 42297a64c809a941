"""Full-size Whisper-large-v3 shapes against vectors recorded from the reference
(fp32 CPU run of the unmodified reference on the same seeded weights and clip):
one 30 s clip, 4-token prompt, 224 greedy tokens with EOS suppressed.

fp32 engine: the 224 token ids must be identical.  bf16 engine: encoder states
within 1e-2 relative L2 and teacher-forced logits within 3e-2 x logit RMS."""
import os

import numpy as np
import pytest
import torch

from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions, TOK_EOT
from whisperdrz_b200.weights import init_state_dict

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def large():
    dims = ModelDimensions.from_name("large-v3")
    return dims, init_state_dict(dims, 0)


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(os.path.join(golden_dir, "model_large_v3_cfg1.npz"))


def _run(e, g, teacher):
    audio = synth.clips([int(s) for s in g["clip_seeds"]])
    xa = e.encode(e.logmel(torch.from_numpy(audio).cuda()))
    logits = e.prefill(xa, [1], [list(map(int, g["prompt"][0]))])
    keep = {int(s): i for i, s in enumerate(g["logit_steps"])}
    stride = int(g["logit_stride"])
    ref_tokens = torch.from_numpy(g["tokens"])
    eot_rule = [{"set_ids": [TOK_EOT]}]  # EOS suppressed, as in the recording
    toks, worst = [], 0.0
    ref_rms = float(torch.from_numpy(g["logits"]).pow(2).mean().sqrt())
    cur = e.rules_argmax(logits, eot_rule)
    for step in range(ref_tokens.shape[1]):
        if step in keep:
            ref = torch.from_numpy(g["logits"][:, keep[step]])
            worst = max(worst, float((logits[:, ::stride].cpu() - ref).abs().max()))
        toks.append(int(cur[0]))
        feed = ref_tokens[:, step] if teacher else cur
        cur, logits = e.decode_step(feed, [1], rules=eot_rule, want_logits=True)
    return xa, toks, worst / ref_rms


def test_large_v3_fp32_tokens_identical(large, golden):
    from whisperdrz_b200.engine import Engine
    dims, sd = large
    e = Engine(dims, sd, dtype=torch.float32, n_slots=3, max_clips=1)
    xa, toks, worst = _run(e, golden, teacher=False)
    gx = torch.from_numpy(golden["xa"])
    assert (xa[:, ::50].float().cpu() - gx).norm() / gx.norm() < 1e-4
    assert toks == [int(t) for t in golden["tokens"][0]]
    assert worst < 1e-3
    assert e.seq_lens()[1] == int(golden["final_seq_lens"][1])
    e.close()


def test_large_v3_bf16_within_tolerance(large, golden):
    from whisperdrz_b200.engine import Engine
    dims, sd = large
    e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=3, max_clips=1)
    xa, toks, worst = _run(e, golden, teacher=True)
    gx = torch.from_numpy(golden["xa"])
    rel = float((xa[:, ::50].float().cpu() - gx).norm() / gx.norm())
    assert rel < 1e-2, rel
    assert worst < 3e-2, worst
    e.close()


@pytest.mark.parametrize("dtype,tol_max,tol_mean,frames", [(torch.float32, 5e-3, 5e-4, 1), (torch.bfloat16, 0.6, 0.03, 75)])
def test_large_v3_word_timing_alignment(large, golden_dir, dtype, tol_max, tol_mean, frames):
    """Word-timing alignment at full size against the reference's recording (tests/golden/make_align_golden.py
    --large: its ten alignment heads, a 44-id chunk with two word anchors on a 30 s clip).  fp32: cost matrix
    (z-scores of order one) within 5e-3 and the word times within one 20 ms frame; bf16 (tcgen05 pass): matrix
    within 0.6 max / 0.03 mean; most word boundaries equal the reference's and none is further than 1.5 s
    (with random weights the cost surface is flat and the path slips between near-equal costs)."""
    from whisperdrz_b200 import alignment as A
    from whisperdrz_b200.engine import Engine
    g = np.load(os.path.join(golden_dir, "align_large.npz"))
    dims, sd = large
    assert [tuple(int(v) for v in h) for h in g["heads"]] == A.ALIGNMENT_HEADS_LARGE_V3
    e = Engine(dims, sd, dtype=dtype, n_slots=2, max_clips=1, max_rows=64)
    audio = synth.clips([int(g["clip_seed"])])
    xa = e.encode(e.logmel(torch.from_numpy(audio).cuda()))
    gx = torch.from_numpy(g["xa_slice"])
    assert float((xa[0, ::50].float().cpu() - gx).norm() / gx.norm()) < (1e-4 if dtype == torch.float32 else 1e-2)
    e.cross_kv(xa, [1])
    e.align_configure(A.ALIGNMENT_HEADS_LARGE_V3)
    ids, word_lens = g["ids"].tolist(), g["word_lens"].tolist()
    tokens, lens = A.build_full_tokens([ids])
    assert lens[0] == int(g["actual_len"])
    cap = int(g["audio_cap"])
    m = e.align_matrix(tokens, lens, [1], [cap]).cpu()
    e.device_status()
    ref = torch.from_numpy(g["matrix_slice"])
    diff = (m[0, : lens[0], :cap][:, ::7] - ref[: lens[0]]).abs()
    assert float(diff.max()) < tol_max and float(diff.mean()) < tol_mean, (float(diff.max()), float(diff.mean()))
    anchors = [(int(a), b, c) for a, b, c in g["word_anchors"].tolist()]
    chunk = A.AlignChunk(slot=1, ids=ids, word_lens=word_lens, num_frames=2 * cap, word_anchors=anchors)
    times = np.array(A.align_chunks(e, [chunk])[0])
    e.device_status()
    want = g["word_times"]
    assert times.shape == want.shape
    assert np.abs(times - want).max() <= 0.02 * frames + 1e-9, (times.tolist(), want.tolist())
    assert np.median(np.abs(times - want)) <= 0.02 + 1e-9              # most boundaries are the reference's own
    e.close()
