"""Test infrastructure: the recorded decode_batch cases of tests/golden/rules_groups.npz
(tests/golden/make_rules_groups_golden.py) as ``RowRules`` + expected blocked set + expected token."""
import os

import numpy as np
import torch

from whisperdrz_b200.decode_rules import RowRules, RuleTables

V = 51866


def steered_logits(seed: int, rows: int, hot: list[int], scale: float) -> torch.Tensor:
    """Same draws as tests/golden/make_rules_groups_golden.py:steered_logits."""
    g = torch.Generator().manual_seed(seed)
    lg = torch.randn(rows, V, generator=g) * scale
    pick = torch.randint(0, len(hot), (rows, 12), generator=g)
    lift = torch.rand(rows, 12, generator=g) * 30.0 + 8.0
    use = torch.rand(rows, generator=g) < 0.8
    for r in range(rows):
        if use[r]:
            lg[r, torch.tensor(hot)[pick[r]]] += lift[r]
    return lg


def load(golden_dir):
    g = np.load(os.path.join(golden_dir, "rules_groups.npz"))
    tables = {}
    for si in range(len(g["settings"])):
        tables[si] = RuleTables.from_arrays({k: g[f"tables{si}_{k}"] for k in
                                             ("names", "bits", "n_vocab", "newline_id", "timing0", "n_timings", "flags")})
    names = g["group_names"].tolist()
    hot = g["hot"].tolist()
    cases = []
    for i in range(len(g["seed"])):
        groups = frozenset(n for n, m in zip(names, g["member"][i]) if m)
        lt = float(g["last_timing"][i])
        rng = tuple(int(v) for v in g["range"][i])
        row = RowRules(groups=groups, language=str(g["lang"][i]) or None, last_timing=None if lt < 0 else lt,
                       bracket_partial=str(g["partial"][i]), timing_range=None if rng[0] < 0 else rng,
                       penalty_ids=tuple(int(t) for t in g["pen"][i] if t >= 0))
        mask = np.unpackbits(g["mask"][i], bitorder="little")[:V].astype(bool)
        cases.append({"setting": int(g["setting"][i]), "row": row, "mask": mask, "token": int(g["token"][i]),
                      "seed": int(g["seed"][i]), "rows": int(g["rows"][i]), "r": int(g["row"][i])})
    return tables, cases, hot, float(g["scale"])
