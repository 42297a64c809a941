"""The fused rule kernel driven by descriptors compiled from the reference's own rule set
(whisperdrz_b200/decode_rules.py): on the logits and group memberships recorded from the reference's
decode_batch (tests/golden/make_rules_groups_golden.py) the device returns the reference's token ids."""
import numpy as np
import pytest
import torch

import rules_cases
from oracle import oracle
from oracle_engine import rule_from_words
from whisperdrz_b200 import decode_rules as R
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.weights import init_state_dict

pytestmark = pytest.mark.gpu


def test_device_rules_return_the_reference_tokens(golden_dir):
    from whisperdrz_b200.engine import Engine
    tables, cases, hot, scale = rules_cases.load(golden_dir)
    dims = ModelDimensions.from_name("test-small")
    sd = init_state_dict(dims, 0)
    for si, t in tables.items():
        mine = [c for c in cases if c["setting"] == si]
        e = Engine(dims, sd, dtype=torch.float32, n_slots=8, max_clips=1, max_rows=64,
                   tables=torch.from_numpy(t.matrix()))
        by_call: dict = {}
        for c in mine:
            by_call.setdefault((c["seed"], c["rows"]), []).append(c)
        for (seed, rows), cs in by_call.items():
            lg = rules_cases.steered_logits(seed, rows, hot, scale)
            sel = lg[[c["r"] for c in cs]].cuda()
            arr = R.compile_rows([c["row"] for c in cs], t)
            got = e.rules_argmax(sel, torch.from_numpy(arr).cuda()).tolist()
            assert got == [c["token"] for c in cs], [sorted(c["row"].groups) for c in cs]
        # the same descriptors inside a decode step: ids must match the oracle's rules on the step's own logits
        rows = [c["row"] for c in mine[:8]]
        arr = R.compile_rows(rows, t)
        xa = torch.randn(1, dims.n_audio_ctx, dims.n_audio_state, generator=torch.Generator().manual_seed(si))
        slots = list(range(len(rows)))
        for s in slots:
            e.cross_kv(xa.cuda(), [s])
        e.slot_reset(slots)
        e.forward_rows([50258] * len(rows), slots, [0] * len(rows), want_logits=False)
        nxt, logits = e.decode_step([50259 + i for i in slots], slots, rules=torch.from_numpy(arr).cuda(), want_logits=True)
        mat = torch.from_numpy(t.matrix())
        want = oracle.rules_argmax(logits.cpu(), [rule_from_words(a) for a in arr], mat)
        assert nxt.tolist() == want.tolist()
        # Phase-4 style re-argmax on the held logits, no penalty (decoding.py:2033-2044)
        re = e.reargmax(slots, torch.from_numpy(arr).cuda()).tolist()
        assert re == oracle.rules_argmax(logits.cpu(), [rule_from_words(a) for a in arr], mat, penalty=False).tolist()
        e.device_status()
        e.close()
