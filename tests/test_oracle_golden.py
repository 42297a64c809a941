"""Pin the CPU oracle against vectors recorded from the reference itself
(tests/golden/make_golden.py).  Runs without a GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions, TOK_EOT
from whisperdrz_b200.weights import init_state_dict


def _mel30(seed, secs):
    a = torch.from_numpy(synth.clip(seed, secs))
    return oracle.window_mel(oracle.log_mel(a))


@pytest.mark.parametrize("name", ["clip30", "clip7", "clip1"])
def test_logmel_matches_reference(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "mel.npz"))
    mel = _mel30(int(g[f"{name}_seed"]), float(g[f"{name}_secs"]))
    assert mel.shape == (128, 3000)
    got = mel[:, ::37].numpy()
    assert np.abs(got - g[f"{name}_mel"]).max() < 2e-4
    assert abs(mel.double().sum().item() - float(g[f"{name}_sum"])) < 1e-2 * 128 * 30


def test_filterbank_shape_and_support():
    fb = oracle.mel_filterbank()
    assert fb.shape == (201, 128)
    assert float(fb[200].abs().max()) == 0.0  # Nyquist row carries no weight
    assert int((fb > 0).sum(0).max()) <= 16


def _run_oracle_model(name, g, n_steps):
    dims = ModelDimensions.from_name(name)
    sd = init_state_dict(dims, int(g["seed"]))
    audio = synth.clips([int(s) for s in g["clip_seeds"]])
    mel = torch.stack([oracle.window_mel(oracle.log_mel(torch.from_numpy(a))) for a in audio])
    xa = oracle.encoder(sd, mel, dims.n_audio_layer, dims.n_audio_head)
    B = xa.shape[0]
    dec = oracle.SlotDecoder(sd, dims.n_text_layer, dims.n_text_head, B + 2, dims.n_text_ctx)
    slots = list(range(1, B + 1))
    logits = dec.prefill(torch.from_numpy(g["prompt"]), xa, slots)[:, -1]
    eot = min(TOK_EOT, dims.n_vocab - 1)
    toks, kept = [], []
    for _ in range(n_steps):
        kept.append(logits[:, :: int(g["logit_stride"])].clone())
        lg = logits.clone()
        lg[:, eot] = float("-inf")
        nxt = lg.argmax(-1)
        toks.append(nxt)
        logits = dec.forward(nxt[:, None], slots)[:, 0]
    return xa, torch.stack(toks, 1), torch.stack(kept, 1), dec


@pytest.mark.parametrize("name,file", [("test-small", "model_test_small.npz"),
                                       ("test-tiny", "model_test_tiny.npz")])
def test_model_matches_reference(golden_dir, name, file):
    g = np.load(os.path.join(golden_dir, file))
    n_steps = g["tokens"].shape[1]
    xa, toks, logits, dec = _run_oracle_model(name, g, n_steps)
    ref_xa = torch.from_numpy(g["xa"])
    rel = (xa[:, ::50] - ref_xa).norm() / ref_xa.norm()
    assert rel < 1e-4, rel
    assert abs((xa.double() ** 2).sum().item() / float(g["xa_sqsum"]) - 1) < 1e-4
    assert np.array_equal(toks.numpy(), g["tokens"])  # fp32: identical greedy ids
    ref_logits = torch.from_numpy(g["logits"])
    assert (logits - ref_logits).abs().max() < 1e-3 * ref_logits.pow(2).mean().sqrt()
    assert np.array_equal(dec.seq_lens.numpy(), g["final_seq_lens"])


def test_rules_argmax_semantics():
    torch.manual_seed(0)
    V = 300
    logits = torch.randn(3, V)
    tables = torch.zeros(2, V, dtype=torch.bool)
    tables[0, :100] = True
    tables[1, 50:250] = True
    rules = [
        {"mode": oracle.MODE_OR, "table_bits": 0b11},               # only 250.. allowed
        {"mode": oracle.MODE_ALL_EXCEPT_RANGE, "arg0": 10, "arg1": 20},
        {"forced_id": 7},
    ]
    out = oracle.rules_argmax(logits, rules, tables)
    assert 250 <= out[0] < 300 and out[0] == 250 + int(logits[0, 250:].argmax())
    assert out[1] == 10 + int(logits[1, 10:20].argmax())
    assert out[2] == 7
    # ties resolve to the lowest index; penalty can move the winner
    lg = torch.zeros(1, V)
    lg[0, 5] = lg[0, 9] = 2.0
    assert oracle.rules_argmax(lg, [{}], tables)[0] == 5
    assert oracle.rules_argmax(lg, [{"pen_ids": [5]}], tables)[0] == 9
    assert oracle.rules_argmax(lg, [{"pen_ids": [5]}], tables, penalty=False)[0] == 5


def _rules_cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "rules_phase34.npz"))
    V = 51866
    cases = []
    for i in range(len(g["seed"])):
        gen = torch.Generator().manual_seed(int(g["seed"][i]))
        lg = torch.randn(int(g["rows"][i]), V, generator=gen) * float(g["scale"])
        mask = torch.from_numpy(np.unpackbits(g["mask"][i], bitorder="little")[:V].astype(bool))
        pen = [int(t) for t in g["pen"][i] if t >= 0]
        cases.append((lg[int(g["row"][i])], mask, pen, int(g["phase"][i]), int(g["token"][i])))
    return cases


def test_rules_argmax_matches_reference_decode_batch(golden_dir):
    """Phase 3 (mask + repetition penalty + argmax) and Phase 4 (re-argmax under
    a new mask, no penalty) of the reference's decode_batch, recorded by
    tests/golden/make_rules_golden.py: same logits, same blocked set, same
    penalised ids -> same token id."""
    cases = _rules_cases(golden_dir)
    assert len(cases) >= 30 and any(c[3] == 4 for c in cases) and any(c[2] for c in cases)
    for lg, mask, pen, phase, tok in cases:
        got = oracle.rules_argmax(lg[None], [{"table_bits": 1, "pen_ids": pen}], mask[None], penalty=phase == 3)
        assert int(got[0]) == tok
