"""Record the reference's Phase-1 group memberships together with the blocked mask its Phase 2 builds.

Run where the reference is mounted:

    PYTHONPATH=<reference>/src python tests/golden/make_rules_groups_golden.py

The unmodified reference ``Transcriber`` runs on a tiny random model under four
settings (tags / emphasis allowed or not, language given or detected).  Its
``decode_batch`` is fed seeded logits that are steered towards structural tokens
(brackets, angle tags, parentheses, emphasis marks, quotes, punctuation, digits,
newline, timestamps), so that the text state machine visits its constraint
groups.  Three methods of the transcriber's ``DecoderState`` object are wrapped
(not changed) to look at ``decode_batch``'s local variables at the moment its
mask is complete: the ``*_indices`` group lists, the per-row contexts and the
finished ``[rows, vocab]`` mask; ``sample_logits`` is wrapped to record the ids
chosen.  Stored per case: settings, group names, language, last timestamp,
bracket prefix, open timestamp range, penalised ids, logit seed and row ->
blocked bitset and token id.  Also stored: the reference's class tables
(``RuleTables.to_arrays``), so that the tests need no tokenizer.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from whisperdrz_b200 import synth  # noqa: E402
from whisperdrz_b200.decode_rules import RuleTables  # noqa: E402
from whisperdrz_b200.dims import ModelDimensions  # noqa: E402
from whisperdrz_b200.weights import init_state_dict  # noqa: E402

import whisperdrz.decoding as ref_dec  # noqa: E402
import whisperdrz.transcriber as ref_tr  # noqa: E402
from whisperdrz.config import Config, ModelDimensions as RefDims  # noqa: E402
from whisperdrz.model import WhisperDRZ  # noqa: E402

V = 51866
SCALE = 4.0
MAX_CASES = 260
SETTINGS = [(False, False, "en"), (True, True, "en"), (True, True, None), (False, False, None)]
EXTRA = {"block_asterisk_combined": "block_asterisk_combined", "block_bracket_after_close": "block_bracket_after_close"}


def steered_logits(seed: int, rows: int, hot: list[int]) -> torch.Tensor:
    """Gaussian rows; in every row a random handful of the structural ids is lifted well above the rest."""
    g = torch.Generator().manual_seed(seed)
    lg = torch.randn(rows, V, generator=g) * SCALE
    pick = torch.randint(0, len(hot), (rows, 12), generator=g)
    lift = torch.rand(rows, 12, generator=g) * 30.0 + 8.0
    use = torch.rand(rows, generator=g) < 0.8
    for r in range(rows):
        if use[r]:
            lg[r, torch.tensor(hot)[pick[r]]] += lift[r]
    return lg


def hot_ids(tok) -> list[int]:
    out = []
    for s in ["[", "]", " [", "<", ">", "(", ")", " (", "*", " *", '"', ' "', ".", ",", "!", "?", "-", "'", " ", "\n",
              "0", "1", "2", "c", "laugh", "pause", "breath", "cut", "cough", "music", " the", " and", "ing", "a",
              "emotion", "accent", ":", "happy", "off", "<|en|>", "<|de|>"]:
        try:
            ids = tok.encode(s)
        except Exception:
            continue
        if len(ids) == 1:
            out.append(int(ids[0]))
    out += [tok.eot] + list(range(tok.timestamp_begin, tok.timestamp_begin + 1501, 37))
    return sorted(set(out))


CRAFTED = [
    "[0] hello", "[0] hello there", "[0] <|1.00|>he (wo", "[0] <|1.00|>hello<|1.50|> (", "[0] <|1.00|>hello<|1.50|> [lau",
    "[0] <|1.00|>hello<|1.50|> [", "[0] <|1.00|>hello<|1.50|> [pause", "[0] <|1.00|>hello <em", "[0] <|1.00|>hello <emotion:happy>",
    '[0] <|1.00|>he said "', "[0] <|1.00|>*wor", "[0] <|1.00|>*word*", "[0] <|1.00|>hello<|1.50|> <|1.60|>wor",
    "[0] <|1.00|>hello.", "[0] <|1.00|>hello,<|1.40|>", "[0] <|28.50|>hello<|29.00|> wor", "[0] <|1.00|>hello<|1.50|> [laugh]",
    "[0] <|1.00|>hello<|1.50|>\n[1] <|2.00|>yes<|2.40|>\n[0] ", "[0] <|1.00|>hello<|1.50|> and ",
]


def crafted_calls(t, tok, tags, stars):
    """A few hand-written text states pushed straight through the (wrapped) decode_batch, for groups the random
    walk above reaches rarely: parentheses, quotes, a line without any timestamp, tag prefixes."""
    from whisperdrz.inference_utils import InferenceState
    for lo in range(0, len(CRAFTED), 4):
        curs = CRAFTED[lo: lo + 4]
        states, last_ids = [], []
        for k, cur in enumerate(curs):
            ids = tok.encode(cur)
            s = InferenceState(index=k, status="started", cur=cur, language="en", meta={"duration": 30.0})
            s.token_count, s.last_token_id, s.recent_tokens = 21, int(ids[-1]), [int(i) for i in ids[-10:]]
            states.append(s)
            last_ids.append(int(ids[-1]))
        ref_tr.decode_batch(torch.zeros(len(curs), V), states, t.ds, temperature=0.0, last_token_ids=last_ids,
                            token_counts=[21] * len(curs), allow_tags=tags, allow_asterisks=stars,
                            speaker_tags=t.speaker_tags, all_tokens_gpu=None, slot_indices=list(range(len(curs))))


def main():
    dims = ModelDimensions(128, 1500, 64, 1, 1, V, 448, 64, 1, 1)
    m = WhisperDRZ(RefDims(**dims.as_dict()), config=Config()).float().eval()
    m.load_state_dict(init_state_dict(dims, 0), strict=False)
    hot = hot_ids(m.tokenizer)
    cases, seen, tables = [], set(), {}
    orig_decode, orig_sample, orig_range = ref_tr.decode_batch, ref_dec.sample_logits, ref_dec._get_timing_range_cpu
    for si, (tags, stars, lang) in enumerate(SETTINGS):
        t = ref_tr.Transcriber(model_path=None, model=m, lang=lang, dtw_align=False, speaker_remap=False, BS=4,
                               allow_tags=tags, allow_asterisks=stars)
        t.load_model(device="cpu")
        ds = t.ds
        tables[si] = RuleTables.from_decoder_state(ds, tags, stars)
        st = {"n": 0, "cur": None, "phase2": False, "ranges": []}
        get_mask, get_add = ds.get_batch_mask_scratch, ds.get_additive_scratch

        def mask_wrap(BS, _f=get_mask):
            st["phase2"], st["ranges"] = True, []
            return _f(BS)

        def add_wrap(BS, dtype, _f=get_add):
            st["phase2"] = False
            loc = sys._getframe(1).f_locals
            if st["cur"] is not None and "batch_mask" in loc:
                groups = {k[: -len("_indices")]: list(v) for k, v in loc.items()
                          if k.endswith("_indices") and isinstance(v, list)}
                for k in EXTRA:
                    groups[k] = list(loc.get(k, []))
                special = loc["special_timing_indices"]
                st["cur"]["snap"] = {
                    "groups": groups, "need": list(loc["need_sampling"]), "forced_close": set(loc["forced_close_indices"]),
                    "contexts": [dict(c) for c in loc["contexts"]],
                    "langs": [getattr(s, "language", None) for s in loc["states"]],
                    "ranges": dict(zip(special, st["ranges"])), "mask": loc["batch_mask"].clone()}
            return _f(BS, dtype)

        def range_wrap(*a, **kw):
            out = orig_range(*a, **kw)
            if st["phase2"]:
                st["ranges"].append((int(out[0]), int(out[1])))
            return out

        def decode_wrap(logits, states, ds_, **kw):
            st["n"] += 1
            seed = 5000 * (si + 1) + st["n"]
            lg = steered_logits(seed, logits.shape[0], hot).to(logits.dtype)
            st["cur"] = {"seed": seed, "rows": logits.shape[0], "logits": lg, "samples": []}
            out = orig_decode(lg, states, ds_, **kw)
            cur, st["cur"] = st["cur"], None
            harvest(cur, si)
            return out

        def sample_wrap(x, temperature=0.0, *a, **kw):
            out = orig_sample(x, temperature, *a, **kw)
            if st["cur"] is not None and temperature == 0.0 and x.dim() == 2:
                st["cur"]["samples"].append((x.detach().clone(), out.detach().clone()))
            return out

        def harvest(cur, si):
            snap = cur.get("snap")
            if snap is None or not cur["samples"]:
                return
            x, out = cur["samples"][0]                       # Phase 3 samples every row of the batch at once
            lg = cur["logits"]
            for i in snap["need"]:
                if i in snap["forced_close"]:
                    continue
                mask = snap["mask"][i]
                base = lg[i] + torch.where(mask, torch.tensor(-65504.0), torch.tensor(0.0))
                pen = torch.nonzero(x[i] != base).flatten().tolist()
                if len(pen) > 10:
                    continue
                names = sorted(k for k, v in snap["groups"].items() if i in v)
                ctx = snap["contexts"][i]
                line = ctx.get("line", "") or ""
                partial = line[line.rfind("[") + 1:] if "in_bracket" in names else ""
                rng = snap["ranges"].get(i)
                key = (si, tuple(names), partial, rng, hash(mask.numpy().tobytes()), tuple(pen))
                if key in seen:
                    continue
                seen.add(key)
                cases.append({"setting": si, "groups": names, "lang": snap["langs"][i] or "",
                              "last_timing": -1.0 if ctx.get("last_timing") is None else float(ctx["last_timing"]),
                              "partial": partial, "range": rng or (-1, -1), "pen": pen, "seed": cur["seed"],
                              "rows": cur["rows"], "row": i, "mask": np.packbits(mask.numpy(), bitorder="little"),
                              "token": int(out[i])})

        ds.get_batch_mask_scratch, ds.get_additive_scratch = mask_wrap, add_wrap
        ref_tr.decode_batch, ref_dec.sample_logits, ref_dec._get_timing_range_cpu = decode_wrap, sample_wrap, range_wrap
        try:
            for k in range(3):
                t.transcribe(torch.from_numpy(synth.long_form(20 + 10 * si + k, 95.0)))
            crafted_calls(t, m.tokenizer, tags, stars)
        finally:
            ref_tr.decode_batch, ref_dec.sample_logits, ref_dec._get_timing_range_cpu = orig_decode, orig_sample, orig_range
        print(f"setting {SETTINGS[si]}: {st['n']} decode_batch calls, {len(cases)} cases so far", flush=True)

    # keep every distinct group combination first, then fill up
    by_combo: dict = {}
    for c in cases:
        by_combo.setdefault((c["setting"], tuple(c["groups"])), []).append(c)
    keep = [v[0] for v in by_combo.values()]
    rest = [c for v in by_combo.values() for c in v[1:]]
    keep += rest[: max(0, MAX_CASES - len(keep))]
    names = sorted({g for c in keep for g in c["groups"]})
    print(f"{len(cases)} cases, {len(by_combo)} group combinations, keeping {len(keep)}; groups seen: {names}")
    pen = np.full((len(keep), 10), -1, np.int64)
    member = np.zeros((len(keep), len(names)), bool)
    for r, c in enumerate(keep):
        pen[r, : len(c["pen"])] = c["pen"]
        member[r, [names.index(g) for g in c["groups"]]] = True
    out = {"scale": np.float64(SCALE), "group_names": np.array(names), "member": member,
           "setting": np.array([c["setting"] for c in keep]), "lang": np.array([c["lang"] for c in keep]),
           "last_timing": np.array([c["last_timing"] for c in keep]), "partial": np.array([c["partial"] for c in keep]),
           "range": np.array([c["range"] for c in keep]), "pen": pen, "seed": np.array([c["seed"] for c in keep]),
           "rows": np.array([c["rows"] for c in keep]), "row": np.array([c["row"] for c in keep]),
           "mask": np.stack([c["mask"] for c in keep]), "token": np.array([c["token"] for c in keep]),
           "hot": np.array(hot), "settings": np.array([[a, b, l is None] for a, b, l in SETTINGS])}
    for c in keep:                                   # base sets of every language a kept case runs under
        tables[c["setting"]].base_tables(c["lang"] or "en")
    for si, tb in tables.items():
        for k, v in tb.to_arrays().items():
            out[f"tables{si}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "rules_groups.npz"), **out)


if __name__ == "__main__":
    main()
