"""CPU-only checks: the C-ABI library builds/loads and exports every symbol the
header declares, and the host-side packing logic is right.  No GPU compute."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from oracle import oracle
from whisperdrz_b200 import capi, frontend
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.weights import init_state_dict, n_params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from whisperdrz_b200 import build
    build.build()
    return capi.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "wdz.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wdz_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    declared = _declared_symbols()
    assert len(declared) >= 18
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in wdz.h but not exported"
        assert name in capi.SYMBOLS, f"{name} has no ctypes prototype"
    assert sorted(capi.SYMBOLS) == declared
    assert b"sm_100a" in lib.wdz_version()


def test_create_validates_config_without_a_gpu(lib):
    dims = ModelDimensions.from_name("test-tiny")
    good = [getattr(dims, f) for f in ("n_mels", "n_audio_ctx", "n_audio_state", "n_audio_head", "n_audio_layer",
                                       "n_vocab", "n_text_ctx", "n_text_state", "n_text_head", "n_text_layer")]
    h = C.c_void_p()
    cfg = capi.Config(*good, capi.WDZ_F32, 4, 64, 1, 64, 0)
    assert lib.wdz_engine_create(C.byref(cfg), C.byref(h)) == capi.WDZ_OK
    need = C.c_size_t()
    assert lib.wdz_workspace_bytes(h, C.byref(need)) == capi.WDZ_OK and need.value > 1 << 20
    # not finalized: compute entry points refuse to run
    assert lib.wdz_encode(h, 1, 1, 1, None) == -4
    assert b"finalized" in lib.wdz_last_error(h)
    assert lib.wdz_engine_destroy(h) == capi.WDZ_OK
    bad = capi.Config(*good, 7, 4, 64, 1, 64, 0)            # unknown dtype
    assert lib.wdz_engine_create(C.byref(bad), C.byref(h)) == -1
    bad = capi.Config(*good, capi.WDZ_F32, 4, 9999, 1, 64, 0)  # cache longer than n_text_ctx
    assert lib.wdz_engine_create(C.byref(bad), C.byref(h)) == -1
    bad_dims = list(good)
    bad_dims[2] = 100                                        # head_dim != 64
    bad = capi.Config(*bad_dims, capi.WDZ_F32, 4, 64, 1, 64, 0)
    assert lib.wdz_engine_create(C.byref(bad), C.byref(h)) == -1


def test_rule_desc_layout_matches_header():
    assert C.sizeof(capi.RuleDesc) == 128
    from whisperdrz_b200.engine import pack_rules
    arr = pack_rules([{"forced_id": 5}, {"mode": 2, "arg0": 3, "arg1": 9, "table_bits": 0x80000001,
                                        "set_ids": [1, 2], "clear_ids": [7], "pen_ids": [4, 4, 6]}])
    w = arr.view(np.int32).reshape(2, 32)
    assert w[0, 0] == 5 and w[1, 0] == -1
    assert list(w[1, 1:4]) == [2, 3, 9] and np.uint32(w[1, 4]) == 0x80000001
    assert w[1, 7] == 2 and list(w[1, 8:10]) == [1, 2]
    assert w[1, 16] == 1 and w[1, 17] == 7
    assert w[1, 21] == 2 and list(w[1, 22:24]) == [4, 6]      # duplicates collapse
    with pytest.raises(ValueError):
        pack_rules([{"set_ids": list(range(9))}])


def test_pack_tables_bit_order():
    from whisperdrz_b200.engine import pack_tables
    V = 70
    t = torch.zeros(2, V, dtype=torch.bool)
    t[0, [0, 31, 32, 69]] = True
    t[1, 5] = True
    p = pack_tables(t, V).numpy().view(np.uint32)
    assert p.shape == (32, 3)
    assert p[0, 0] == (1 | 1 << 31) and p[0, 1] == 1 and p[0, 2] == 1 << 5
    assert p[1, 0] == 1 << 5 and p[2:].sum() == 0


def test_frontend_tables_match_oracle_filterbank():
    fb, lo, hi = frontend.mel_filterbank(128)
    ref = oracle.mel_filterbank(201, 128).numpy()
    assert np.abs(fb - ref).max() < 1e-6
    for m in range(128):
        assert fb[: lo[m], m].sum() == 0 and fb[hi[m]:, m].sum() == 0
    w = frontend.hann_periodic()
    assert np.abs(w - torch.hann_window(400).numpy()).max() < 1e-6
    tw = frontend.twiddle()
    assert tw.shape == (400, 2) and abs(tw[100, 1] - 1.0) < 1e-7


def test_weight_packing_shapes_and_param_count():
    from whisperdrz_b200.engine import pack_weights
    dims = ModelDimensions.from_name("test-tiny")
    sd = init_state_dict(dims, 0)
    packed = pack_weights(sd, dims, torch.float32, "cpu")
    d = dims.n_text_state
    assert packed["decoder.cross_kv.weight"].shape == (dims.n_text_layer * 2 * d, d)
    assert packed["encoder.blocks.0.attn.qkv.bias"][d: 2 * d].abs().sum() == 0   # key has no bias
    w = sd["encoder.conv1.weight"]
    assert torch.equal(packed["encoder.conv1.weight"][:, dims.n_mels: 2 * dims.n_mels], w[:, :, 1])
    big = ModelDimensions.from_name("large-v3")
    # parameter count of large-v3 from shapes alone (1 541 570 560)
    da, dt = big.n_audio_state, big.n_text_state
    blk = lambda dd, cross: (4 * dd * dd + 3 * dd + 2 * dd) * (2 if cross else 1) + 8 * dd * dd + 5 * dd + 2 * dd
    total = (da * big.n_mels * 3 + da + da * da * 3 + da + big.n_audio_layer * blk(da, False) + 2 * da
             + big.n_vocab * dt + big.n_text_ctx * dt + big.n_text_layer * blk(dt, True) + 2 * dt)
    assert total == 1541570560
    assert n_params(sd) > 0


def test_engine_refuses_to_run_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name("test-tiny")
    with pytest.raises(RuntimeError):
        Engine(dims, {}, dtype=torch.float32)


def test_gelu_fast_polynomial_as_written_in_the_kernel_source():
    """The branch-free GELU of the bf16 tensor-core epilogues (``csrc/common.cuh: gelu_fast``): the coefficients are
    read out of the CUDA source, the formula is restated in float32 numpy, and the result is held against
    0.5 x (1 + erf(x / sqrt 2)) in float64 over the whole range - the bound the header comment and the design state."""
    from scipy.special import erf
    src = open(os.path.join(ROOT, "whisperdrz_b200", "csrc", "common.cuh")).read()
    body = src[src.index("float gelu_fast(float x)"):]
    body = body[:body.index("\n}\n")]
    first = re.search(r"float q = (-?[0-9.e+-]+)f;", body).group(1)
    rest = re.findall(r"q = fmaf\(q, a, (-?[0-9.e+-]+)f\);", body)
    coef = [np.float32(first)] + [np.float32(c) for c in rest]
    assert len(coef) == 7 and "fminf(fabsf(z), 4.0f)" in body
    f = np.float32
    x = np.linspace(-12.0, 12.0, 1_200_001).astype(f)
    z = (x * f(0.70710678118654752440)).astype(f)
    a = np.minimum(np.abs(z), f(4.0))
    q = np.full_like(a, coef[0])
    for c in coef[1:]:
        q = (q * a + c).astype(f)
    e = np.exp2((-q * a).astype(f)).astype(f)
    er = np.copysign((f(1.0) - e).astype(f), z)
    h = (f(0.5) * x).astype(f)
    got = (h * er + h).astype(f).astype(np.float64)
    xd = x.astype(np.float64)
    ref = 0.5 * xd * (1.0 + erf(xd / np.sqrt(2.0)))
    assert np.abs(er.astype(np.float64) - erf(z.astype(np.float64))).max() < 2.5e-7      # erf itself, exact 2^x
    assert np.abs(got - ref).max() < 1e-6                                                  # the GELU value
