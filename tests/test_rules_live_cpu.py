"""The rule binding against the LIVE reference (oracle/_ref): the reference's own ``decode_batch`` runs on
hand-written text states; at the moment its blocked mask is complete its local variables are read (through a
wrapper around a ``DecoderState`` method it calls there), handed to ``decode_rules.rows_from_decode_batch`` exactly as
a maintainer's binding would, and the compiled descriptors must stand for the reference's mask bit for bit."""
import sys

import pytest
import torch

from oracle import oracle, ref
from whisperdrz_b200 import decode_rules as R
from oracle_engine import rule_from_words

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref is not installed")

V = 51866
STATES = [
    "[0] hello", "[0] <|1.00|>he (wo", "[0] <|1.00|>hello<|1.50|> [lau", "[0] <|1.00|>hello<|1.50|> [",
    "[0] <|1.00|>hello <em", '[0] <|1.00|>he said "', "[0] <|1.00|>*wor", "[0] <|1.00|>hello<|1.50|> <|1.60|>wor",
    "[0] <|1.00|>hello.", "[0] <|1.00|>hello,<|1.40|>", "[0] <|28.50|>hello<|29.00|> wor", "[0] <|1.00|>hello<|1.50|> [laugh]",
    "[0] <|1.00|>hello<|1.50|>\n[1] <|2.00|>yes<|2.40|>\n[0] ", "[0] <|1.00|>hello<|1.50|> and ", "[0] <|1.00|>hello<|1.50|>",
    "[0] <|1.00|>", "[", "[0] <|1.00|>hello<|1.50|> <|1.60|>",
]


@pytest.mark.parametrize("tags,stars", [(False, False), (True, True)])
def test_binding_reproduces_the_live_reference(tags, stars):
    ref.load()
    import whisperdrz.decoding as D
    from whisperdrz.inference_utils import InferenceState, init_for_model
    from whisperdrz.tokenizer import get_tokenizer

    tok = get_tokenizer(True, num_languages=100, language="en")

    class M:        # what init_for_model reads
        tokenizer = tok

        class dims:
            n_vocab = V
    init_for_model(M)
    ds = D.DecoderState(tok, device="cpu")
    ds.init_gpu_tensors()
    tables = R.RuleTables.from_decoder_state(ds, tags, stars)
    mat = torch.from_numpy(tables.matrix())
    snap = {}
    get_mask, get_add, get_range = ds.get_batch_mask_scratch, ds.get_additive_scratch, D._get_timing_range_cpu

    def mask_wrap(BS):
        snap["ranges"], snap["phase2"] = [], True
        return get_mask(BS)

    def add_wrap(BS, dtype):
        loc = dict(sys._getframe(1).f_locals)
        snap["phase2"] = False
        snap["rows"] = R.rows_from_decode_batch(loc, timing_ranges=dict(zip(loc["special_timing_indices"], snap["ranges"])))
        snap["need"] = list(loc["need_sampling"])
        snap["mask"] = loc["batch_mask"].clone()
        return get_add(BS, dtype)

    def range_wrap(*a, **kw):
        out = get_range(*a, **kw)
        if snap.get("phase2"):
            snap["ranges"].append((int(out[0]), int(out[1])))
        return out

    ds.get_batch_mask_scratch, ds.get_additive_scratch, D._get_timing_range_cpu = mask_wrap, add_wrap, range_wrap
    checked, seen_groups = 0, set()
    try:
        for lo in range(0, len(STATES), 6):
            curs = STATES[lo: lo + 6]
            states, last = [], []
            for k, cur in enumerate(curs):
                ids = tok.encode(cur)
                s = InferenceState(index=k, status="started", cur=cur, language="en", meta={"duration": 30.0})
                s.token_count, s.last_token_id, s.recent_tokens = 21, int(ids[-1]), [int(i) for i in ids[-10:]]
                states.append(s)
                last.append(int(ids[-1]))
            g = torch.Generator().manual_seed(100 + lo)
            logits = torch.randn(len(curs), V, generator=g) * 4.0
            snap.pop("rows", None)
            D.decode_batch(logits.clone(), states, ds, temperature=0.0, last_token_ids=last,
                                 token_counts=[21] * len(curs), allow_tags=tags, allow_asterisks=stars, speaker_tags=True,
                                 all_tokens_gpu=None, slot_indices=list(range(len(curs))))
            if "rows" not in snap:
                continue                                          # every row of this call was decided on the host
            arr = R.compile_rows(snap["rows"], tables)
            for row, i, words in zip(snap["rows"], snap["need"], arr):
                rule = rule_from_words(words)
                got = oracle.blocked_mask(rule, mat, V)
                assert torch.equal(got, snap["mask"][i]), (curs[i], sorted(row.groups))
                seen_groups |= row.groups
                checked += 1
    finally:
        ds.get_batch_mask_scratch, ds.get_additive_scratch, D._get_timing_range_cpu = get_mask, get_add, get_range
    assert checked >= 10
    assert {"normal", "in_bracket", "last_was_timing"} <= seen_groups
