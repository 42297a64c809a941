"""Record what the reference's decode_batch does to logits (Phase 3 and Phase 4).

Run where the reference is mounted:

    PYTHONPATH=<reference>/src python tests/golden/make_rules_golden.py

The unmodified reference Transcriber runs on a tiny random model; two of its
functions are wrapped (not changed): ``decode_batch`` as imported by the
transcriber gets its logits replaced by seeded Gaussian rows, and
``sample_logits`` records every tensor it is asked to sample from together with
the ids it returns.  From the seeded logits and the recorded tensor the blocked
set and the penalised ids of each row are recovered exactly, so each stored
case is (logit seed, row, blocked bitset, penalised ids, phase) -> token id the
reference chose.  Cases with distinct blocked sets are kept (about 40).
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

import whisperdrz.decoding as ref_dec  # noqa: E402
import whisperdrz.transcriber as ref_tr  # noqa: E402
from whisperdrz.config import Config, ModelDimensions as RefDims  # noqa: E402
from whisperdrz.model import WhisperDRZ  # noqa: E402

V = 51866
SCALE = 4.0
MAX_CASES = 40


def seeded_logits(seed: int, rows: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, V, generator=g) * SCALE


def main():
    dims = ModelDimensions(128, 1500, 64, 1, 1, V, 448, 64, 1, 1)
    m = WhisperDRZ(RefDims(**dims.as_dict()), config=Config()).float().eval()
    m.load_state_dict(init_state_dict(dims, 0), strict=False)
    t = ref_tr.Transcriber(model_path=None, model=m, lang="en", dtw_align=False, speaker_remap=False, BS=4)

    calls = []          # one entry per decode_batch call
    state = {"n": 0, "cur": None}
    orig_decode, orig_sample = ref_tr.decode_batch, ref_dec.sample_logits

    def decode_wrap(logits, states, ds, **kw):
        state["n"] += 1
        seed = 1000 + state["n"]
        lg = seeded_logits(seed, logits.shape[0]).to(logits.dtype)
        state["cur"] = {"seed": seed, "rows": logits.shape[0], "logits": lg, "samples": []}
        out = orig_decode(lg, states, ds, **kw)
        calls.append(state["cur"])
        state["cur"] = None
        return out

    def sample_wrap(x, temperature=0.0, *a, **kw):
        out = orig_sample(x, temperature, *a, **kw)
        if state["cur"] is not None and temperature == 0.0 and x.dim() == 2:
            state["cur"]["samples"].append((x.detach().clone(), out.detach().clone()))
        return out

    ref_tr.decode_batch = decode_wrap
    ref_dec.sample_logits = sample_wrap
    try:
        t.transcribe(torch.from_numpy(synth.long_form(7, 100.0)))
    finally:
        ref_tr.decode_batch, ref_dec.sample_logits = orig_decode, orig_sample

    cases, seen = [], set()
    for c in calls:
        lg = c["logits"]
        for k, (x, out) in enumerate(c["samples"]):
            for j in range(x.shape[0]):
                if k == 0:
                    i = j                                # Phase 3 samples every row of the batch
                else:                                    # Phase 4: find the source row by exact matches
                    i = int(((x[j][None] == lg).sum(1)).argmax())
                blocked = (x[j] - lg[i]) < -30000.0
                base = lg[i] + torch.where(blocked, torch.tensor(-65504.0), torch.tensor(0.0))
                pen = torch.nonzero(x[j] != base).flatten().tolist()
                if k > 0 and pen:
                    continue                             # not a clean Phase-4 row
                if len(pen) > 10 or blocked.all():
                    continue
                key = (hash(blocked.numpy().tobytes()), tuple(pen), k > 0)
                if key in seen:
                    continue
                seen.add(key)
                cases.append({"seed": c["seed"], "rows": c["rows"], "row": i, "phase": 4 if k > 0 else 3,
                              "mask": np.packbits(blocked.numpy(), bitorder="little"), "pen": pen,
                              "token": int(out[j]), "n_blocked": int(blocked.sum())})
    # keep a spread of blocked-set sizes, Phase-4 cases first
    cases.sort(key=lambda c: (c["phase"] != 4, c["n_blocked"]))
    p4 = [c for c in cases if c["phase"] == 4][:10]
    p3 = [c for c in cases if c["phase"] == 3]
    step = max(1, len(p3) // (MAX_CASES - len(p4)))
    keep = p4 + p3[::step][: MAX_CASES - len(p4)]
    print(f"{len(calls)} decode_batch calls, {len(cases)} distinct cases, keeping {len(keep)} "
          f"({len(p4)} phase 4); blocked sizes {sorted(c['n_blocked'] for c in keep)}")
    pen = np.full((len(keep), 10), -1, np.int64)
    for r, c in enumerate(keep):
        pen[r, : len(c["pen"])] = c["pen"]
    np.savez_compressed(
        os.path.join(HERE, "rules_phase34.npz"), scale=np.float64(SCALE),
        seed=np.array([c["seed"] for c in keep]), rows=np.array([c["rows"] for c in keep]),
        row=np.array([c["row"] for c in keep]), phase=np.array([c["phase"] for c in keep]),
        mask=np.stack([c["mask"] for c in keep]), pen=pen, token=np.array([c["token"] for c in keep]))


if __name__ == "__main__":
    main()
