"""GPU parity: the CUDA engine, called through the C ABI, against the CPU
oracle and the golden vectors recorded from the reference.

Tolerances: fp32 engine - greedy token ids identical, logits within 1e-3 of
logit RMS, encoder states within 1e-4 relative L2; bf16 engine - teacher-forced
logits within 3e-2 x logit RMS (max-abs), encoder states within 1e-2 relative
L2; log-mel within 1e-3 max-abs; rule/argmax results identical.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions, TOK_EOT
from whisperdrz_b200.weights import init_state_dict

pytestmark = pytest.mark.gpu

F32_LOGIT_TOL = 1e-3
BF16_LOGIT_TOL = 3e-2
F32_ENC_TOL = 1e-4
BF16_ENC_TOL = 1e-2
MEL_TOL = 1e-3


def _engine(name, dtype, seed=0, **kw):
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name(name)
    sd = init_state_dict(dims, seed)
    return Engine(dims, sd, dtype=dtype, **kw), dims, sd


@pytest.fixture(scope="module")
def small_f32():
    e, dims, sd = _engine("test-small", torch.float32, n_slots=6, max_clips=3)
    yield e, dims, sd
    e.close()


@pytest.fixture(scope="module")
def small_bf16():
    e, dims, sd = _engine("test-small", torch.bfloat16, n_slots=6, max_clips=3)
    yield e, dims, sd
    e.close()


def _oracle_mel(audio_np):
    return torch.stack([oracle.window_mel(oracle.log_mel(torch.from_numpy(a))) for a in audio_np])


# --------------------------------------------------------------------------- mel
def test_logmel_matches_oracle_and_golden(small_f32, golden_dir):
    e, _, _ = small_f32
    g = np.load(os.path.join(golden_dir, "mel.npz"))
    for name in ("clip30", "clip7", "clip1"):
        a = synth.clip(int(g[f"{name}_seed"]), float(g[f"{name}_secs"]))
        buf = torch.zeros(1, 480000)
        buf[0, : len(a)] = torch.from_numpy(a)
        mel = e.logmel(buf.cuda(), n_samples=[len(a)]).cpu()[0]
        ref = oracle.window_mel(oracle.log_mel(torch.from_numpy(a)))
        assert (mel - ref).abs().max() < MEL_TOL
        assert np.abs(mel[:, ::37].numpy() - g[f"{name}_mel"]).max() < MEL_TOL


def test_logmel_ragged_batch_and_window_offset(small_f32):
    e, _, _ = small_f32
    lens = [480000, 123456, 16000]
    buf = torch.zeros(3, 480000)
    clips = [synth.clip(20 + i, n / 16000) for i, n in enumerate(lens)]
    for i, c in enumerate(clips):
        buf[i, : len(c)] = torch.from_numpy(c)
    offs = [0, 250, 40]
    mel = e.logmel(buf.cuda(), n_samples=lens, frame_offset=offs).cpu()
    for i, c in enumerate(clips):
        ref = oracle.window_mel(oracle.log_mel(torch.from_numpy(c)), offs[i])
        assert (mel[i] - ref).abs().max() < MEL_TOL
        n_valid = max(0, lens[i] // 160 - offs[i])
        assert torch.all(mel[i, :, n_valid:] == -1.5)


# ----------------------------------------------------------------------- encoder
def _encoder_case(e, dims, sd, seeds, tol, golden=None):
    audio = synth.clips(seeds)
    mel_ref = _oracle_mel(audio)
    xa_ref = oracle.encoder(sd, mel_ref, dims.n_audio_layer, dims.n_audio_head)
    mel = e.logmel(torch.from_numpy(audio).cuda())
    xa = e.encode(mel).float().cpu()
    rel = (xa - xa_ref).norm() / xa_ref.norm()
    assert rel < tol, rel
    if golden is not None:
        gx = torch.from_numpy(golden["xa"])
        assert (xa[:, ::50] - gx).norm() / gx.norm() < tol
    return xa_ref


def test_encoder_f32(small_f32, golden_dir):
    e, dims, sd = small_f32
    g = np.load(os.path.join(golden_dir, "model_test_small.npz"))
    _encoder_case(e, dims, sd, [int(s) for s in g["clip_seeds"]], F32_ENC_TOL, g)


def test_encoder_bf16(small_bf16, golden_dir):
    e, dims, sd = small_bf16
    g = np.load(os.path.join(golden_dir, "model_test_small.npz"))
    _encoder_case(e, dims, sd, [int(s) for s in g["clip_seeds"]], BF16_ENC_TOL, g)


# ----------------------------------------------------------------------- decoder
def _greedy(e, dims, xa, prompt, slots, n_steps, teacher=None):
    """Prefill + n_steps; returns (tokens [B, n_steps], logits [B, n_steps, V]).
    With ``teacher`` ([B, n_steps]) the fed tokens are the teacher's."""
    eot = min(TOK_EOT, dims.n_vocab - 1)
    logits = e.prefill(xa, slots, [list(map(int, p)) for p in prompt])
    toks, kept = [], []
    for step in range(n_steps):
        kept.append(logits.cpu())
        lg = logits.clone()
        lg[:, eot] = float("-inf")
        nxt = lg.argmax(-1)
        toks.append(nxt.cpu())
        feed = nxt if teacher is None else torch.as_tensor(teacher[:, step]).cuda()
        _, logits = e.decode_step(feed, slots, rules=None, want_logits=True)
    return torch.stack(toks, 1), torch.stack(kept, 1)


def test_decoder_f32_tokens_identical_to_reference(small_f32, golden_dir):
    e, dims, sd = small_f32
    g = np.load(os.path.join(golden_dir, "model_test_small.npz"))
    audio = synth.clips([int(s) for s in g["clip_seeds"]])
    xa = e.encode(e.logmel(torch.from_numpy(audio).cuda()))
    B, n_steps = g["tokens"].shape
    slots = list(range(1, B + 1))
    toks, logits = _greedy(e, dims, xa, g["prompt"], slots, n_steps)
    assert np.array_equal(toks.numpy(), g["tokens"])
    ref = torch.from_numpy(g["logits"])
    got = logits[:, :, :: int(g["logit_stride"])]
    assert (got - ref).abs().max() < F32_LOGIT_TOL * ref.pow(2).mean().sqrt()
    sl = e.seq_lens()
    assert sl[1: B + 1] == [int(v) for v in g["final_seq_lens"][1: B + 1]]


def test_decoder_bf16_teacher_forced_logits(small_bf16, golden_dir):
    e, dims, sd = small_bf16
    g = np.load(os.path.join(golden_dir, "model_test_small.npz"))
    audio = synth.clips([int(s) for s in g["clip_seeds"]])
    xa = e.encode(e.logmel(torch.from_numpy(audio).cuda()))
    B, n_steps = g["tokens"].shape
    _, logits = _greedy(e, dims, xa, g["prompt"], list(range(1, B + 1)), n_steps, teacher=g["tokens"])
    ref = torch.from_numpy(g["logits"])
    got = logits[:, :, :: int(g["logit_stride"])]
    assert (got - ref).abs().max() < BF16_LOGIT_TOL * ref.pow(2).mean().sqrt()


def test_ragged_rows_against_oracle(small_f32):
    """Slots at different depths with prompts of different lengths, decoded in
    one packed step per iteration, against the oracle run slot by slot."""
    e, dims, sd = small_f32
    rng = np.random.default_rng(7)
    audio = synth.clips([11, 12])
    mel = _oracle_mel(audio)
    xa_ref = oracle.encoder(sd, mel, dims.n_audio_layer, dims.n_audio_head)
    xa = xa_ref.cuda()
    prompts = [list(rng.integers(0, 50000, 9)), list(rng.integers(0, 50000, 4))]
    slots = [4, 2]
    dec = oracle.SlotDecoder(sd, dims.n_text_layer, dims.n_text_head, 6, dims.n_text_ctx)
    dec.set_cross(xa_ref, slots)
    dec.reset(slots)
    ref_last = [dec.forward(torch.tensor([p]), [s])[0, -1] for p, s in zip(prompts, slots)]
    got = e.prefill(xa, slots, prompts).cpu()
    rms = torch.stack(ref_last).pow(2).mean().sqrt()
    assert (got - torch.stack(ref_last)).abs().max() < F32_LOGIT_TOL * rms
    assert [e.seq_lens()[s] for s in slots] == [9, 4]
    cur = got.argmax(-1)
    for _ in range(5):
        ref = torch.stack([dec.forward(cur[i].view(1, 1), [s])[0, 0] for i, s in enumerate(slots)])
        nxt, lg = e.decode_step(cur, slots, want_logits=True)
        assert (lg.cpu() - ref).abs().max() < F32_LOGIT_TOL * rms
        assert torch.equal(nxt.cpu().long(), ref.argmax(-1))
        cur = ref.argmax(-1)
    assert [e.seq_lens()[s] for s in slots] == [14, 9]
    # a slot that was reset starts again at position 0 and leaves the other alone
    e.slot_reset([2])
    assert e.seq_lens()[2] == 0 and e.seq_lens()[4] == 14


# ------------------------------------------------------------------------- rules
def test_rules_argmax_bit_exact():
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name("test-tiny")
    sd = init_state_dict(dims, 0)
    V = dims.n_vocab
    g = torch.Generator().manual_seed(3)
    tables = torch.rand(5, V, generator=g) < 0.3
    e = Engine(dims, sd, dtype=torch.float32, n_slots=16, max_clips=1, tables=tables)
    logits = torch.randn(12, V, generator=g) * 3
    logits[5, 100] = logits[5, 7] = 50.0            # tie -> lowest id
    rules = [
        {},
        {"table_bits": 0b10101},
        {"mode": oracle.MODE_ALL_EXCEPT_TABLE, "arg0": 1, "table_bits": 0b1},
        {"mode": oracle.MODE_ALL_EXCEPT_RANGE, "arg0": 900, "arg1": 1200},
        {"mode": oracle.MODE_ALL, "clear_ids": [3, 77, 1500]},
        {},
        {"prefix_begin": 0, "prefix_end": 1000, "set_ids": [1001, 1002], "clear_ids": [5]},
        {"forced_id": 42},
        {"pen_ids": [int(logits[8].argmax())]},
        {"pen_ids": list(map(int, logits[9].topk(10).indices))},
        {"table_bits": 0b11111, "pen_ids": [1, 2, 3]},
        {"mode": oracle.MODE_ALL},                   # everything blocked: plain argmax of shifted row
    ]
    ref = oracle.rules_argmax(logits, rules, tables)
    got = e.rules_argmax(logits.cuda(), rules).cpu().long()
    assert torch.equal(got, ref)
    ref2 = oracle.rules_argmax(logits, rules, tables, penalty=False)
    got2 = e.rules_argmax(logits.cuda(), rules, penalty=False).cpu().long()
    assert torch.equal(got2, ref2)
    assert got[5] == 7
    e.device_status()
    # a NaN row is reported, not silently argmax-ed
    bad = logits.clone()
    bad[0, 10] = float("nan")
    out = e.rules_argmax(bad.cuda(), rules).cpu()
    assert out[0] == -1
    from whisperdrz_b200.capi import WdzError
    with pytest.raises(WdzError):
        e.device_status()
    e.device_status()  # cleared by the read
    e.close()


def test_capacity_and_argument_errors(small_f32):
    from whisperdrz_b200.capi import WdzError
    e, dims, _ = small_f32
    with pytest.raises(WdzError):
        e.encode(torch.zeros(4, dims.n_mels, 3000))          # > max_clips
    with pytest.raises(WdzError):
        e.decode_step([1] * 100, [0] * 100)                  # > max_rows
    with pytest.raises(ValueError):
        e.logmel(torch.zeros(1, 300))                        # too short to reflect-pad


# ------------------------------------------------------------------- tcgen05 GEMM
@pytest.mark.parametrize("M,N,K,gelu", [(128, 256, 64, False), (300, 512, 256, True), (3000, 1280, 384, True),
                                        (1500, 3840, 1280, False), (777, 1280, 5120, False)])
def test_tensor_core_linear_matches_fp32_reference(small_bf16, M, N, K, gelu):
    """tcgen05 GEMM against a plain fp32 product of the same bf16-rounded
    operands; tolerance = bf16 output rounding (2^-8 relative) plus fp32
    accumulation-order noise."""
    e, _, _ = small_bf16
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = (torch.randn(N, generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T + b.float()
    if gelu:
        ref = torch.nn.functional.gelu(ref)
    got = e.linear(x, w, b, gelu=gelu).float().cpu()
    e.device_status()
    err = (got - ref).abs().max() / ref.abs().max()
    assert err < 6e-3, err
    got_cc = e.linear(x, w, b, gelu=gelu, cuda_cores_only=True).float().cpu()
    assert (got - got_cc).abs().max() / ref.abs().max() < 6e-3
    # the CTA-pair kernel (M > 128) and the lone-CTA kernel add the same k-blocks in the same order
    got_lone = e.linear(x, w, b, gelu=gelu, cuda_cores_only=2).float().cpu()
    e.device_status()
    assert torch.equal(got, got_lone)


def test_tensor_core_gelu_epilogue_against_exact_erf(small_bf16):
    """The branch-free GELU of the tensor-core epilogues against 0.5 x (1 + erf(x / sqrt 2)) in float64: a 0/1 weight
    matrix makes every output gelu(x[m, k]) of one bf16 input exactly, so what is left is the epilogue's own error
    (below 1e-6 absolute) and the final rounding to bf16 (2^-9 relative)."""
    e, _, _ = small_bf16
    M, K, N = 512, 64, 256
    x = torch.linspace(-9.0, 9.0, M * K).reshape(M, K).bfloat16()
    w = torch.zeros(N, K)
    w[torch.arange(N), torch.arange(N) % K] = 1.0
    xd = x.double()[:, torch.arange(N) % K]
    ref = 0.5 * xd * (1.0 + torch.erf(xd / 2.0 ** 0.5))
    for mode in (0, 2):
        got = e.linear(x, w.bfloat16(), None, gelu=True, cuda_cores_only=mode).double().cpu()
        e.device_status()
        err = (got - ref).abs()
        assert bool((err <= ref.abs() * 2.0 ** -8 + 1.5e-6).all()), float((err - ref.abs() * 2.0 ** -8).max())
        # and it lands on the correctly rounded bf16 value wherever the value is not itself of the size of that error
        big = ref.abs() >= 1e-3
        assert (got[big] != ref.float().bfloat16().double()[big]).double().mean() < 0.005


def test_split_decode_step_matches_the_unsplit_step():
    """A step of 352 rows runs as two half-batches on two streams; with ``FLAG_NO_SPLIT_STEP`` it runs as one batch.
    Same kernels on the same operands, only the K-split partial sums arrive in another order: the logits agree within
    bf16 order noise (2e-2 x RMS, the bound used between the two product kernels below), over a prompt pass and two
    single-token steps, and the split engine launches about twice as many kernels per step."""
    from whisperdrz_b200 import capi
    n = 352
    e, dims, sd = _engine("test-small", torch.bfloat16, n_slots=n, max_clips=4, max_rows=2 * n)
    e2, _, _ = _engine("test-small", torch.bfloat16, n_slots=n, max_clips=4, max_rows=2 * n, flags=capi.FLAG_NO_SPLIT_STEP)
    rng = np.random.default_rng(5)
    audio = torch.from_numpy(synth.clips([41, 42, 43, 44])).cuda()
    slots = list(range(n))
    first = [int(t) for t in rng.integers(0, 50000, n)]
    out, counts = [], []
    for eng in (e, e2):
        xa = eng.encode(eng.logmel(audio))
        for i in range(0, n, 4):
            eng.cross_kv(xa, slots[i: i + 4])
        eng.slot_reset(slots)
        steps = []
        tok = first
        for pos in range(3):
            before = eng.launch_count()
            lg = eng.forward_rows(tok, slots, [pos] * n, emit_rows=list(range(n)))
            counts.append(eng.launch_count() - before)
            steps.append(lg.float().cpu())
            tok = [int(t) for t in steps[-1].argmax(-1)] if eng is e else [int(t) for t in out[0][pos].argmax(-1)]
        eng.device_status()
        out.append(steps)
    for a, b in zip(out[0], out[1]):
        rms = b.pow(2).mean().sqrt()
        assert (a - b).abs().max() < 2e-2 * rms
    assert counts[0] > 1.8 * counts[3]          # split: every layer kernel once per half
    e.close(); e2.close()


def test_decoder_bf16_many_rows_tensor_core_path():
    """More than 16 token rows per call take the operand-swapped tcgen05 product
    (prefill of ~150 prompt rows, then decode steps over 20 slots at different
    depths).  Two checks: (1) it agrees with the mma.sync path of the same
    engine (same bf16 operands, fp32 accumulation; bf16 re-rounding of the
    activations between layers amplifies order noise: within 2e-2 x logit RMS);
    (2) both stay within 5e-2 x logit RMS of the fp32 oracle - the max is taken
    over 20 rows x 51866 logits of a 2-layer random model fed random prompt
    ids, where bf16 rounding of weights alone gives 3-4e-2 on either path."""
    from whisperdrz_b200 import capi
    e, dims, sd = _engine("test-small", torch.bfloat16, n_slots=24, max_clips=2, max_rows=256)
    e2, _, _ = _engine("test-small", torch.bfloat16, n_slots=24, max_clips=2, max_rows=256,
                       flags=capi.FLAG_NO_TENSOR_CORE)
    rng = np.random.default_rng(11)
    audio = synth.clips([31, 32])
    mel = _oracle_mel(audio)
    xa_ref = oracle.encoder(sd, mel, dims.n_audio_layer, dims.n_audio_head)
    n = 20
    slots = list(range(2, 2 + n))
    xa_rows = xa_ref[[i % 2 for i in range(n)]]
    prompts = [list(map(int, rng.integers(0, 50000, int(rng.integers(3, 13))))) for _ in range(n)]
    dec = oracle.SlotDecoder(sd, dims.n_text_layer, dims.n_text_head, 24, dims.n_text_ctx)
    dec.set_cross(xa_rows, slots)
    dec.reset(slots)
    ref = torch.stack([dec.forward(torch.tensor([p]), [s])[0, -1] for p, s in zip(prompts, slots)])
    tok, sl, pos, emit = [], [], [], []
    for p, s in zip(prompts, slots):
        for j, t in enumerate(p):
            tok.append(t); sl.append(s); pos.append(j)
        emit.append(len(tok) - 1)
    assert len(tok) > 100
    rms = ref.pow(2).mean().sqrt()
    got = []
    for eng in (e, e2):
        for i in range(0, n, 2):   # at most max_clips windows per cross-K/V call
            eng.cross_kv(xa_rows[i: i + 2].cuda(), slots[i: i + 2])
        eng.slot_reset(slots)
        got.append(eng.forward_rows(tok, sl, pos, emit_rows=emit).cpu())
    assert (got[0] - got[1]).abs().max() < 2e-2 * rms
    assert (got[0] - ref).abs().max() < 5e-2 * rms
    cur = ref.argmax(-1)
    for _ in range(3):
        ref = torch.stack([dec.forward(cur[i].view(1, 1), [s])[0, 0] for i, s in enumerate(slots)])
        _, lg = e.decode_step(cur, slots, want_logits=True)
        _, lg2 = e2.decode_step(cur, slots, want_logits=True)
        assert (lg - lg2).abs().max().cpu() < 2e-2 * rms
        assert (lg.cpu() - ref).abs().max() < 5e-2 * rms
        cur = ref.argmax(-1)
    e.device_status()
    assert [e.seq_lens()[s] for s in slots] == [len(p) + 3 for p in prompts]
    e.close()
    e2.close()


def test_tensor_core_encoder_attention_matches_fp32_reference(small_bf16):
    """tcgen05 flash attention (S and PV on the tensor cores, P through TMEM)
    against softmax(q k^T / 8) v in fp32 on the same bf16 inputs.  Tolerance:
    bf16 rounding of P and of the output (2^-8 relative each)."""
    e, dims, _ = small_bf16
    g = torch.Generator().manual_seed(5)
    B, T, d, H = 2, dims.n_audio_ctx, dims.n_audio_state, dims.n_audio_head
    qkv = torch.randn(B, T, 3 * d, generator=g)
    qkv[..., :d] *= 2.0          # sharper softmax than unit-variance scores
    qkv = qkv.bfloat16()
    q, k, v = (t.float().view(B, T, H, 64).permute(0, 2, 1, 3) for t in qkv.split(d, dim=-1))
    ref = torch.softmax(q @ k.transpose(-1, -2) / 8.0, -1) @ v
    ref = ref.permute(0, 2, 1, 3).reshape(B, T, d)
    got = e.encoder_attention(qkv).float().cpu()
    e.device_status()
    err = (got - ref).abs().max() / ref.abs().max()
    assert err < 1.5e-2, err
    assert (got - ref).norm() / ref.norm() < 6e-3
    got_cc = e.encoder_attention(qkv, cuda_cores_only=True).float().cpu()
    assert (got_cc - ref).abs().max() / ref.abs().max() < 1.5e-2


def test_drop_in_model_follows_the_reference_call_sequence(golden_dir):
    """B200Model driven exactly as the reference Transcriber drives its model
    (create_flash_kv, reset_flash_kv, encoder, prefill_flash, forward_flash with
    positions read from self_kv[0].seq_lens) reproduces the reference recording."""
    from whisperdrz_b200.model import B200Model
    g = np.load(os.path.join(golden_dir, "model_test_small.npz"))
    dims = ModelDimensions.from_name("test-small")
    m = B200Model(dims, init_state_dict(dims, int(g["seed"])), dtype=torch.float32).cuda().eval()
    B, n_steps = g["tokens"].shape
    self_kv, cross_kv = m.create_flash_kv(B + 2, max_tokens=dims.n_text_ctx)
    slots = torch.arange(1, B + 1, device="cuda")
    m.reset_flash_kv(self_kv, cross_kv, slots)
    m.decoder.cache_embedding_weight(torch.float32)
    audio = synth.clips([int(s) for s in g["clip_seeds"]])
    mel = m.engine.logmel(torch.from_numpy(audio).cuda())
    xa = m.encoder(mel)
    logits = m.prefill_flash(torch.from_numpy(g["prompt"]).cuda(), xa, self_kv, cross_kv, slots)[:, -1]
    eot = TOK_EOT
    toks = []
    for _ in range(n_steps):
        lg = logits.clone()
        lg[:, eot] = float("-inf")
        nxt = lg.argmax(-1)
        toks.append(nxt.cpu())
        pos = self_kv[0].seq_lens[slots]
        logits = m.decoder.forward_flash(nxt[:, None], self_kv, cross_kv, pos, slot_indices=slots)[:, 0]
    assert np.array_equal(torch.stack(toks, 1).numpy(), g["tokens"])
    assert np.array_equal(self_kv[0].seq_lens.cpu().numpy()[1: B + 1], g["final_seq_lens"][1: B + 1])
    m.engine.close()


def test_rules_kernel_matches_reference_decode_batch(golden_dir):
    """The device rule kernel on the cases recorded from the reference's own
    decode_batch (tests/golden/make_rules_golden.py): identical token ids for
    Phase 3 (with penalty) and Phase 4 (re-argmax, no penalty)."""
    from test_oracle_golden import _rules_cases
    from whisperdrz_b200.engine import Engine
    cases = _rules_cases(golden_dir)
    dims = ModelDimensions.from_name("test-small")
    sd = init_state_dict(dims, 0)
    for lo in range(0, len(cases), 32):
        part = cases[lo: lo + 32]
        tables = torch.stack([c[1] for c in part])
        e = Engine(dims, sd, dtype=torch.float32, n_slots=2, max_clips=1, tables=tables)
        logits = torch.stack([c[0] for c in part]).cuda()
        rules = [{"table_bits": 1 << i, "pen_ids": c[2]} for i, c in enumerate(part)]
        with_pen = e.rules_argmax(logits, rules, penalty=True).cpu().tolist()
        no_pen = e.rules_argmax(logits, rules, penalty=False).cpu().tolist()
        for i, c in enumerate(part):
            assert (with_pen[i] if c[3] == 3 else no_pen[i]) == c[4], (lo + i, c[3])
        e.close()


def test_transcribe_end_to_end_identical_to_oracle_scheduler():
    """The whole path behind ``Transcriber.transcribe`` - chunking, slot refill,
    log-mel, encoder, prefill, rule-constrained greedy decode, a continuation
    window, stitching - on the fp32 CUDA engine against the same scheduler
    driven by the CPU oracle: identical tokens, segments and stop reasons."""
    from oracle_engine import OracleEngine
    from whisperdrz_b200.engine import Engine
    from whisperdrz_b200.rules import timestamp_tables
    from whisperdrz_b200.transcriber import Transcriber
    dims = ModelDimensions.from_name("test-small")
    sd = init_state_dict(dims, 0)
    audio = torch.from_numpy(synth.long_form(5, 71.0))           # 3 chunks, the last one 11 s
    kw = dict(max_new_tokens=20, max_continuations=1)
    ref_tr = Transcriber(OracleEngine(dims, sd, n_slots=2, max_clips=2), **kw)
    ref_tr._rules_dev = lambda a: torch.from_numpy(a)
    want = ref_tr.transcribe(audio)
    e = Engine(dims, sd, dtype=torch.float32, n_slots=2, max_clips=2, tables=timestamp_tables(dims.n_vocab))
    # rule state on the device (several steps per host round trip) and on the host (one step per round trip)
    for mode in (dict(device_rules=True, steps_per_poll=5), dict(device_rules=False)):
        got = Transcriber(e, **kw, **mode).transcribe(audio)
        e.device_status()
        assert [r["id"] for r in got.raw_chunks] == ["chunk_0", "chunk_1", "chunk_2"]
        for a, b in zip(got.raw_chunks, want.raw_chunks):
            assert a["tokens"] == b["tokens"], mode
            assert a["stop_reason"] == b["stop_reason"] and a["windows"] == b["windows"]
        assert got.segments == want.segments and len(got.segments) >= 3
        assert any(r["windows"] == 2 for r in got.raw_chunks)    # the continuation path ran
    e.close()


def test_load_model_entry_point_and_warm_slots():
    """``whisperdrz_b200.load_model`` (the shape of the reference's ``whisperdrz.load_model``,
    __init__.py:9-22) gives a ready Transcriber; with a warm pool (log-mel, encoder and cross K/V of the next
    chunks on a side stream, event-gated promotion) it returns the tokens of the plain scheduler."""
    import whisperdrz_b200
    audio = torch.from_numpy(synth.long_form(6, 100.0))          # 4 chunks
    kw = dict(dtype=torch.float32, max_clips=2, max_new_tokens=16, max_continuations=0, dtw_align=True,
              align_heads=[(0, 1), (1, 0), (1, 3)])
    plain = whisperdrz_b200.load_model("test-small", n_slots=2, **kw)
    want = plain.transcribe(audio)
    plain.engine.device_status()
    assert [r["id"] for r in want.raw_chunks] == [f"chunk_{i}" for i in range(4)]
    assert all(r["tokens"] and r["stop_reason"] in ("eot", "max_tokens") for r in want.raw_chunks)
    assert all("word_times" in r for r in want.raw_chunks)      # dtw_align=True: token-level word timing
    plain.engine.close()
    warm = whisperdrz_b200.load_model("test-small", n_slots=4, n_warm=2, **kw)
    got = warm.transcribe(audio)
    warm.engine.device_status()
    assert warm.promoted == 4 and warm.prefill_stream is not None
    assert [r["tokens"] for r in got.raw_chunks] == [r["tokens"] for r in want.raw_chunks]
    assert [r["word_times"] for r in got.raw_chunks] == [r["word_times"] for r in want.raw_chunks]
    warm.engine.close()


@pytest.mark.parametrize("M,N", [(1, 1280), (8, 1280), (16, 1280), (40, 1280), (256, 1280), (300, 1280),
                                 (100, 1280), (200, 1280), (200, 3840), (129, 5120), (72, 2000)])
def test_decode_shaped_linear_matches_fp32_reference(small_bf16, M, N):
    """wdz_linear_rows: the mma.sync weight-streaming kernel (<= 16 rows) and the
    operand-swapped tcgen05 kernel (more rows: ragged row tiles, K splits, feature
    counts that are no multiple of 128, chunks above 256 rows) against an fp32
    product of the same bf16 operands, storing and accumulating."""
    e, _, _ = small_bf16
    g = torch.Generator().manual_seed(M)
    K = 1024
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = (torch.randn(N, generator=g) * 0.1).bfloat16()
    ref = x.float() @ w.float().T + b.float()
    got = e.linear_rows(x, w, b).cpu()
    assert (got - ref).abs().max() / ref.abs().max() < 2e-5
    acc = torch.full((M, N), 0.5, device="cuda")
    e.linear_rows(x, w, b, out=acc)
    assert (acc.cpu() - (ref + 0.5)).abs().max() / ref.abs().max() < 2e-5
    e.device_status()


def test_device_rule_state_through_the_abi(small_f32):
    """wdz_ts_*: reset, first token, k queued steps, poll and token log against
    the host rule state driving wdz_decode_step one step at a time."""
    from whisperdrz_b200 import rules as R
    from whisperdrz_b200.transcriber import rules_to_array
    e, dims, sd = small_f32
    # the fixture engine has no class tables: build one that has them
    from whisperdrz_b200.engine import Engine
    eng = Engine(dims, sd, dtype=torch.float32, n_slots=4, max_clips=2, tables=R.timestamp_tables(dims.n_vocab))
    audio = synth.clips([51, 52])
    xa = eng.encode(eng.logmel(torch.from_numpy(audio).cuda()))
    prompt = [[50258, 50259, 50360]] * 2
    budgets = [9, 30]
    # host rules, one step per call
    slots = [1, 3]
    logits = eng.prefill(xa, slots, prompt)
    rows = [R.RowState(max_new=b) for b in budgets]
    cur = eng.rules_argmax(logits, torch.from_numpy(rules_to_array([r.rule() for r in rows])).cuda()).tolist()
    for r, t in zip(rows, cur):
        r.update(t)
    while not all(r.done for r in rows):
        act = [i for i, r in enumerate(rows) if not r.done]
        nxt = eng.decode_step([rows[i].tokens[-1] for i in act], [slots[i] for i in act],
                              rules=torch.from_numpy(rules_to_array([rows[i].rule() for i in act])).cuda()).tolist()
        for i, t in zip(act, nxt):
            rows[i].update(t)
    # device rules: everything queued, finished rows drop out on the device
    logits = eng.prefill(xa, slots, prompt)
    eng.ts_reset(slots, budgets)
    eng.ts_first(logits, slots)
    eng.ts_steps(slots, 7)
    st = eng.ts_poll()
    assert st[1, 0] == 9 and st[1, 1] == 8 and st[1, 6] == 0          # 1 + 7 tokens, not done yet
    eng.ts_steps(slots, 40)                                            # more than either slot needs
    st = eng.ts_poll()
    for i, s in enumerate(slots):
        assert st[s, 6] == 1 and st[s, 1] == len(rows[i].tokens)
        assert eng.ts_tokens(s, int(st[s, 1])) == rows[i].tokens
    # a finished slot stops growing its KV: length = prompt + generated tokens that were fed back
    lens = eng.seq_lens()
    assert [lens[s] for s in slots] == [3 + len(r.tokens) - 1 for r in rows]
    eng.device_status()
    eng.close()


def test_decode_to_the_last_cache_position(small_f32):
    """One slot decoded until the self-attention cache is full (448 positions:
    every split of the ragged attention, the last cache row, the position
    table's last row), against the oracle; then the engine must refuse nothing
    and keep the slot length at the cache size."""
    e, dims, sd = small_f32
    audio = synth.clips([61])
    mel = _oracle_mel(audio)
    xa_ref = oracle.encoder(sd, mel, dims.n_audio_layer, dims.n_audio_head)
    dec = oracle.SlotDecoder(sd, dims.n_text_layer, dims.n_text_head, 6, dims.n_text_ctx)
    ref = dec.prefill(torch.tensor([[50258, 50259, 50360]]), xa_ref, [5])[:, -1]
    got = e.prefill(xa_ref.cuda(), [5], [[50258, 50259, 50360]])
    rms = ref.pow(2).mean().sqrt()
    cur = ref.argmax(-1)
    worst = float((got.cpu() - ref).abs().max() / rms)
    for step in range(3, dims.n_text_ctx):
        ref = dec.forward(cur.view(1, 1), [5])[:, 0]
        nxt, lg = e.decode_step(cur, [5], want_logits=True)
        if step % 37 == 0 or step >= dims.n_text_ctx - 2:
            worst = max(worst, float((lg.cpu() - ref).abs().max() / rms))
            assert int(nxt[0]) == int(ref.argmax(-1))
        cur = ref.argmax(-1)
    assert worst < F32_LOGIT_TOL, worst
    assert e.seq_lens()[5] == dims.n_text_ctx
    e.device_status()
