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
