"""The reference's rule set compiled into descriptors (whisperdrz_b200/decode_rules.py) against what the
reference's own decode_batch built: for every recorded row, the blocked set that the descriptor stands for
equals the reference's finished mask bit for bit, and the oracle's masked, penalised arg-max returns the
token the reference sampled."""
import numpy as np
import torch

import rules_cases
from oracle import oracle
from whisperdrz_b200 import decode_rules as R


def test_every_mask_step_of_the_reference_is_covered(golden_dir):
    _, cases, _, _ = rules_cases.load(golden_dir)
    seen = set().union(*(c["row"].groups for c in cases))
    # one group per ordered mask step of decode_batch's Phase 2 (decoding.py:1527-1713)
    for name in ("block_open_angle", "block_angle_consecutive", "block_asterisk_combined", "block_star_after_star",
                 "block_space_in_asterisk", "block_timing_in_asterisk", "block_eot", "block_newline", "block_cut",
                 "block_bracket_after_close", "lang", "line_start_digit", "last_was_timing", "last_was_timing_even",
                 "last_was_timing_even_first_word", "last_was_timing_even_timed_tag", "last_was_timing_odd",
                 "last_was_space", "block_punct_nonalnum", "block_quote", "in_bracket", "not_in_bracket", "in_angle",
                 "not_in_angle", "in_asterisk", "in_paren", "not_in_paren", "even_timings_not_after_timing",
                 "last_char_punct_or_bracket", "block_open_bracket", "allow_space_asterisk", "force_timing",
                 "force_timestamp", "line_start_timing", "close_bracket_even_timing"):
        assert name in seen, name
    assert any(c["row"].last_timing and "normal" in c["row"].groups for c in cases)      # backwards-timestamp prefix


def test_compiled_descriptor_reproduces_the_reference_mask_and_token(golden_dir):
    tables, cases, hot, scale = rules_cases.load(golden_dir)
    mats = {si: torch.from_numpy(t.matrix()) for si, t in tables.items()}
    logits = {}
    assert len(cases) >= 200
    for c in cases:
        t = tables[c["setting"]]
        ops = R.row_ops(c["row"], t)
        assert np.array_equal(R.simulate(ops, t), c["mask"]), sorted(c["row"].groups)      # the op list is right
        rule = R.compile_row(c["row"], t)
        got = oracle.blocked_mask(rule, mats[c["setting"]], t.n_vocab).numpy()
        assert np.array_equal(got, c["mask"]), (sorted(c["row"].groups), rule)            # and so is its normal form
        key = (c["seed"], c["rows"])
        if key not in logits:
            logits = {key: rules_cases.steered_logits(c["seed"], c["rows"], hot, scale)}
        tok = oracle.rules_argmax(logits[key][c["r"]][None], [rule], mats[c["setting"]])
        assert int(tok[0]) == c["token"], (sorted(c["row"].groups), int(tok[0]), c["token"])


def test_descriptor_array_layout_round_trips(golden_dir):
    tables, cases, _, _ = rules_cases.load(golden_dir)
    rows = [c["row"] for c in cases if c["setting"] == 1][:40]
    arr = R.compile_rows(rows, tables[1])
    assert arr.shape == (len(rows), 32) and arr.dtype == np.int32
    from oracle_engine import rule_from_words
    mat = torch.from_numpy(tables[1].matrix())
    for a, r in zip(arr, rows):
        want = oracle.blocked_mask(R.compile_row(r, tables[1]), mat, tables[1].n_vocab)
        assert torch.equal(oracle.blocked_mask(rule_from_words(a), mat, tables[1].n_vocab), want)
