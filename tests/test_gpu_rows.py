"""The batched ragged decode at full size (Whisper-large-v3 shapes) against the
reference's own recording (tests/golden/make_golden.py --large-rows): 32 slots
with prompts of 4..420 tokens, 24 teacher-forced decode steps.

These are the configurations the throughput benchmark (384 rows per step) and
the 32-slot decode case run: more than 16 rows per step take the operand-swapped tcgen05 products with
K splits, the split cross-attention query product, the multi-way split
cross-attention and the captured step graph.

Tolerances.  fp32: greedy token ids identical, logits within 1e-3 x RMS.
bf16: every comparison here takes the maximum over 32 rows x 535 logits, and at
that sample size rounding the WEIGHTS to bf16 alone - all arithmetic in fp32,
measured below with the fp32 engine as a control - already gives a max-abs of
3.1-3.3e-2 x the row's logit RMS (RMS error 0.80e-2).  So the bound is stated as:
99.8 % of the logits within 3e-2 x RMS, none beyond 5e-2, RMS error at most
1.1e-2, and the engine's RMS error at most 1.25 x the control's."""
import os

import numpy as np
import pytest
import torch

from whisperdrz_b200.dims import ModelDimensions, TOK_EOT
from whisperdrz_b200.rules import BatchRuleState, timestamp_tables
from whisperdrz_b200.weights import init_state_dict

pytestmark = pytest.mark.gpu

BF16_LOGIT_TOL = 3e-2          # 99.8 % of the logits
BF16_LOGIT_CAP = 5e-2          # every logit
BF16_RMS_TOL = 1.1e-2
N_ROWS = 32
REPLICAS = 12                  # 384 rows per step, what the throughput benchmark batches per GPU


def rows_inputs(n_rows: int = N_ROWS, seed: int = 2):
    """Same draws as tests/golden/make_golden.py:rows_inputs."""
    from whisperdrz_b200 import synth
    _, _, prompts = synth.decode_lengths(seed, n_rows)
    rng = np.random.default_rng(seed + 1)
    for j, n in enumerate((150, 250, 350, 420)):
        prompts[n_rows - 4 + j] = rng.integers(0, 50000, n).astype(np.int64)
    return prompts


def rows_xa(i: int, d: int) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(100 + i)
    return torch.empty(1500, d, dtype=torch.float32).normal_(0.0, 1.0, generator=g)


@pytest.fixture(scope="module")
def large():
    dims = ModelDimensions.from_name("large-v3")
    return dims, init_state_dict(dims, 0)


@pytest.fixture(scope="module")
def golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "model_large_v3_rows.npz"))
    prompts = rows_inputs()
    assert [len(p) for p in prompts] == [int(n) for n in g["prompt_lens"]]
    return g, prompts


def _prefill(e, dims, prompts, slot0: int = 0):
    """Cross K/V + prompt rows of the 32 recorded slots, 8 windows per call; returns the last-prompt-token logits."""
    out = []
    for g0 in range(0, N_ROWS, 8):
        xa = torch.stack([rows_xa(r, dims.n_audio_state) for r in range(g0, g0 + 8)]).cuda()
        out.append(e.prefill(xa, [slot0 + r for r in range(g0, g0 + 8)],
                             [[int(t) for t in prompts[r]] for r in range(g0, g0 + 8)]))
    return torch.cat(out)


def _errors(logits, g, step, stride):
    """|logits - recorded| / recorded row RMS, [replicas, 32, 535]; row r is compared with recorded row r % 32."""
    ref = torch.from_numpy(g["logits"][:, step])
    rms = torch.from_numpy(g["rms"][:, step]).float()
    got = logits[:, ::stride].float().cpu()
    reps = got.shape[0] // N_ROWS
    return (got.view(reps, N_ROWS, -1) - ref[None]).abs() / rms[None, :, None]


def _worst(logits, g, step, stride):
    return float(_errors(logits, g, step, stride).max())


def _check_bf16(logits, g, step, stride, what):
    err = _errors(logits, g, step, stride)
    assert float(err.max()) < BF16_LOGIT_CAP, (what, step, float(err.max()))
    assert float((err < BF16_LOGIT_TOL).float().mean()) >= 0.998, (what, step)
    rms = float(err.pow(2).mean().sqrt())
    assert rms < BF16_RMS_TOL, (what, step, rms)
    return rms


def _replicate(e, prompts, n_copies):
    """Slots 32.. become copies of the prefilled slots 0..31 (caches and lengths)."""
    for j in range(1, n_copies + 1):
        lo = N_ROWS * j
        for t in (e.self_k, e.self_v, e.cross_k, e.cross_v):
            t[:, lo: lo + N_ROWS].copy_(t[:, :N_ROWS])
        e.seq_lens_dev[lo: lo + N_ROWS] = e.seq_lens_dev[:N_ROWS]


def test_large_v3_bf16_ragged_rows_32_and_384(large, golden):
    """(1) 32 ragged rows per step and (2) 384 rows per step (the 32 recorded slots replicated twelve times:
    every replica must reproduce its recorded row) through wdz_prefill + the wdz_decode_step graph."""
    from whisperdrz_b200.engine import Engine
    dims, sd = large
    g, prompts = golden
    stride = int(g["stride"])
    steps = g["tokens"].shape[1] - 1
    e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=N_ROWS * (1 + REPLICAS), max_clips=8, max_rows=2048,
               tables=timestamp_tables(dims.n_vocab))
    logits0 = _prefill(e, dims, prompts)
    rms_err = [_check_bf16(logits0, g, 0, stride, "prefill")]
    assert e.seq_lens()[:N_ROWS] == [len(p) for p in prompts]
    _replicate(e, prompts, REPLICAS)
    fed = torch.from_numpy(g["tokens"])
    slots32 = list(range(N_ROWS))
    slots_big = list(range(N_ROWS, N_ROWS * (1 + REPLICAS)))
    for step in range(steps):
        _, lg = e.decode_step(fed[:, step], slots32, want_logits=True)
        rms_err.append(_check_bf16(lg, g, step + 1, stride, "32 rows"))
        _, lg = e.decode_step(fed[:, step].repeat(REPLICAS), slots_big, want_logits=True)
        _check_bf16(lg, g, step + 1, stride, "384 rows")
    e.device_status()
    lens = e.seq_lens()
    assert lens[:N_ROWS] == [len(p) + steps for p in prompts]
    assert lens[N_ROWS:] == lens[:N_ROWS] * REPLICAS

    # (3) rule state kept on the device (wdz_ts_first / wdz_ts_steps, several steps per host round trip) at
    # 384 rows against the same engine stepped from the host with the same token-level rules: rewind the
    # slots to their prompts and decode 8 tokens each way.  The bf16 step is not bit-reproducible (K-split
    # partial sums meet in fp32 atomics, and a last-bit difference can flip a bf16 rounding further down),
    # so a free-running row now and then takes another of two near-equal logits - replicas of one row do
    # that within a single run, too.  Required: the first token of every row agrees (it comes from the same prefill
    # logits), 95 % of the rows agree on the first two and at least 80 % on all eight (a wrong slot, position or
    # rule on either path would leave none).
    n_new = 8
    lens0 = torch.tensor([len(p) for p in prompts] * (1 + REPLICAS), dtype=torch.int32).cuda()
    first = logits0.repeat(REPLICAS, 1)

    def host_path():
        e.seq_lens_dev.copy_(lens0)
        rs = BatchRuleState(N_ROWS * (1 + REPLICAS), n_new)
        toks = {s: [] for s in slots_big}
        active = list(slots_big)
        cur = e.rules_argmax(first, torch.from_numpy(rs.rules_array(np.asarray(active))).cuda()).tolist()
        for i in range(n_new):
            done = rs.update(np.asarray(active), cur)
            for s, t in zip(active, cur):
                toks[s].append(int(t))
            keep = [j for j, d in enumerate(done) if not d]
            active, cur = [active[j] for j in keep], [cur[j] for j in keep]
            if not active or i == n_new - 1:
                break
            cur = e.decode_step(cur, active, rules=torch.from_numpy(rs.rules_array(np.asarray(active))).cuda()).tolist()
        return toks

    def device_path():
        e.seq_lens_dev.copy_(lens0)
        e.ts_reset(slots_big, [n_new] * len(slots_big))
        e.ts_first(first, slots_big)
        e.ts_steps(slots_big, 3)
        e.ts_steps(slots_big, n_new - 3 - 1)
        st = e.ts_poll()
        return {s: e.ts_tokens(s, int(st[s][1])) for s in slots_big}

    a, b = host_path(), device_path()
    assert all(a[s][:1] == b[s][:1] for s in slots_big)                                # same logits, same rule: no slack
    assert sum(a[s][:2] == b[s][:2] for s in slots_big) >= 0.95 * len(slots_big)
    assert sum(a[s] == b[s] for s in slots_big) >= 0.8 * len(slots_big)
    assert all(len(b[s]) == n_new or b[s][-1] == TOK_EOT for s in slots_big)
    e.device_status()
    e.close()
    del e
    torch.cuda.empty_cache()

    # control: the same weights rounded to bf16, every operation in fp32 (the fp32 engine)
    c = Engine(dims, {k: v.bfloat16().float() for k, v in sd.items()}, dtype=torch.float32, n_slots=N_ROWS,
               max_clips=8, max_rows=2048)
    lg = _prefill(c, dims, prompts)
    floor = [float(_errors(lg, g, 0, stride).pow(2).mean().sqrt())]
    for step in range(6):
        _, lg = c.decode_step(fed[:, step], slots32, want_logits=True)
        floor.append(float(_errors(lg, g, step + 1, stride).pow(2).mean().sqrt()))
    c.close()
    assert np.mean(rms_err[: len(floor)]) <= 1.25 * np.mean(floor), (rms_err[: len(floor)], floor)


def test_large_v3_fp32_ragged_rows_tokens_identical(large, golden):
    """fp32 engine, free-running greedy decode of the 32 ragged rows with EOS suppressed: the 25 token ids of
    every row equal the reference's."""
    from whisperdrz_b200.engine import Engine
    dims, sd = large
    g, prompts = golden
    stride = int(g["stride"])
    steps = g["tokens"].shape[1] - 1
    e = Engine(dims, sd, dtype=torch.float32, n_slots=N_ROWS, max_clips=8, max_rows=2048)
    logits = _prefill(e, dims, prompts)
    rule = [{"set_ids": [TOK_EOT]}] * N_ROWS
    cur = e.rules_argmax(logits, rule)
    toks = [cur.cpu()]
    worst = _worst(logits, g, 0, stride)
    for step in range(steps):
        cur, logits = e.decode_step(cur, list(range(N_ROWS)), rules=rule, want_logits=True)
        toks.append(cur.cpu())
        worst = max(worst, _worst(logits, g, step + 1, stride))
    e.device_status()
    assert np.array_equal(torch.stack(toks, 1).numpy(), g["tokens"])
    assert worst < 1e-3, worst
    e.close()
