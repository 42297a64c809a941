"""The engine behind the reference's own scheduler.

The UNMODIFIED reference ``Transcriber`` (installed into oracle/_ref by
oracle/make_ref.py) runs the same long-form audio twice: once over the
reference model on the CPU (fp32, its SDPA path) and once over
``B200Model`` + ``dropin.bind`` on the GPU.  Chunking, ``decode_batch`` with its
text rules, the stop rules, continuation windows, ``[CHOP]`` stitching and the
clean-up chain are the reference's code in both runs; only the device work
differs.  In fp32 the transcripts must be identical, chunk by chunk.
"""
import re

import numpy as np
import pytest
import torch

from oracle import ref
from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.weights import init_state_dict

pytestmark = pytest.mark.gpu

SECONDS = 75.0      # three chunks: 30 s + 30 s + 15 s


@pytest.fixture(scope="module")
def refmod():
    m = ref.load()
    if m is None:
        pytest.skip("oracle/_ref is not installed (python oracle/make_ref.py where the reference is mounted)")
    return m


@pytest.fixture(scope="module")
def small():
    dims = ModelDimensions.from_name("test-small")
    return dims, init_state_dict(dims, 0)


def _cpu_transcriber(refmod, dims, sd, **kw):
    from whisperdrz.transcriber import Transcriber
    t = Transcriber(model_path=None, model=ref.model(dims, sd), lang="en", speaker_remap=False, BS=4, **kw)
    t.load_model(device="cpu")
    return t


def _b200_transcriber(refmod, dims, sd, dtype=torch.float32, logmel=False, bind=True, **kw):
    from whisperdrz.transcriber import Transcriber
    from whisperdrz_b200 import dropin
    from whisperdrz_b200.model import B200Model
    tok = ref.model(dims, sd).tokenizer
    model = B200Model(dims, sd, dtype=dtype, tokenizer=tok, max_clips=4)
    t = Transcriber(model_path=None, model=model, lang="en", speaker_remap=False, BS=4, **kw)
    if bind:
        dropin.bind(t, logmel=logmel)
    return t


def _chunks(res):
    return [(r["id"], r.get("prediction"), r.get("stop_reason")) for r in res.raw_chunks]


@pytest.fixture(scope="module")
def audio():
    return torch.from_numpy(synth.long_form(11, SECONDS))


@pytest.fixture(scope="module")
def cpu_result(refmod, small, audio):
    dims, sd = small
    return _cpu_transcriber(refmod, dims, sd, dtw_align=False).transcribe(audio)


def test_reference_transcriber_over_engine_gives_identical_text(refmod, small, audio, cpu_result):
    dims, sd = small
    assert len(cpu_result.raw_chunks) == 3
    assert len(cpu_result.text) > 500 and all(r.get("stop_reason") for r in cpu_result.raw_chunks)
    t = _b200_transcriber(refmod, dims, sd, dtw_align=False)
    got = t.transcribe(audio)
    t.model.engine.device_status()
    assert _chunks(got) == _chunks(cpu_result)
    assert got.text == cpu_result.text
    assert got.segments == cpu_result.segments
    assert sum(t.cuda_graphs.hits.values()) > 20          # decode went through the engine's captured step


def test_engine_logmel_under_the_reference_scheduler(refmod, small, audio, cpu_result):
    """Same run with the reference's CPU log-mel module swapped for the engine's kernels
    (mel within 1e-3 of the reference's): same chunk structure and stop reasons, same text."""
    dims, sd = small
    t = _b200_transcriber(refmod, dims, sd, logmel=True, dtw_align=False)
    got = t.transcribe(audio)
    assert [c[0] for c in _chunks(got)] == [c[0] for c in _chunks(cpu_result)]
    assert got.text == cpu_result.text


def test_bf16_engine_under_the_reference_scheduler(refmod, small, audio, cpu_result):
    """The bf16 engine (tcgen05 products and attention, the path the benchmark times) behind the same reference
    scheduler: every chunk comes back with a stop reason and text in the reference's line format (the tokens
    themselves may take the other of two near-equal logits in bf16, after which a free-running transcript of
    a random-weight model differs from the fp32 one)."""
    dims, sd = small
    t = _b200_transcriber(refmod, dims, sd, dtype=torch.bfloat16, logmel=True, dtw_align=False)
    got = t.transcribe(audio)
    t.model.engine.device_status()
    assert [r["id"] for r in got.raw_chunks] == [r["id"] for r in cpu_result.raw_chunks]
    assert all(r.get("stop_reason") and r.get("prediction") for r in got.raw_chunks)
    assert got.text.startswith("[0] <|") and cpu_result.text.startswith("[0] <|")
    assert sum(t.cuda_graphs.hits.values()) > 20


def test_model_seam_alone_without_bind(refmod, small, audio, cpu_result):
    """``Transcriber(model=B200Model(...))`` with nothing else touched: the reference computes log-mel on the CPU
    and, where flash-attn is importable, captures ``forward_flash`` into its bucketed CUDA graphs (the capture then
    holds the engine's kernels).  Its bucket padding re-runs stale rows - the reference's own hazard, which
    ``bind`` removes - so only the structure of the result is checked here."""
    dims, sd = small
    t = _b200_transcriber(refmod, dims, sd, bind=False, dtw_align=False)
    got = t.transcribe(audio)
    t.model.engine.device_status()
    assert [r["id"] for r in got.raw_chunks] == [r["id"] for r in cpu_result.raw_chunks]
    assert all(r.get("stop_reason") and "prediction" in r for r in got.raw_chunks)


def test_forward_flash_inside_a_cuda_graph(refmod, small):
    """The reference captures ``decoder.forward_flash`` into CUDA graphs when flash-attn is importable
    (transcriber.py:91-119).  Captured and replayed, the engine's step gives the logits of a direct call."""
    from whisperdrz_b200.model import B200Model
    dims, sd = small
    m = B200Model(dims, sd, dtype=torch.float32, tokenizer=object(), max_clips=2)
    self_kv, cross_kv = m.create_flash_kv(4, max_tokens=dims.n_text_ctx)
    dev = m.device
    g = torch.Generator().manual_seed(3)
    xa = torch.randn(2, dims.n_audio_ctx, dims.n_audio_state, generator=g).to(dev)
    prompt = torch.tensor([[50258, 50259, 50360, 58], [50258, 50259, 50360, 220]], device=dev)
    slots = torch.tensor([1, 3], device=dev)
    m.prefill_flash(prompt, xa, self_kv, cross_kv, slots)
    tok = torch.tensor([[15], [60]], device=dev)
    static_tok, static_pos, static_slots = tok.clone(), self_kv[0].seq_lens[slots].long(), slots.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = m.decoder.forward_flash(static_tok, self_kv, cross_kv, static_pos, slot_indices=static_slots)
    lens_before = m.engine.seq_lens()
    graph.replay()
    torch.cuda.synchronize()
    captured = static_out.clone()
    assert m.engine.seq_lens()[1] == lens_before[1] + 1
    # rewind the two slots and run the same step directly (the engine's own graph)
    m.engine.seq_lens_dev.copy_(torch.tensor(lens_before, dtype=torch.int32))
    direct = m.decoder.forward_flash(tok, self_kv, cross_kv, static_pos, slot_indices=slots)
    m.engine.device_status()
    rms = float(direct.float().pow(2).mean().sqrt())
    assert float((captured.float() - direct.float()).abs().max()) < 1e-4 * rms
    m.engine.close()


def test_large_v3_bf16_dropin_runs_faster_than_real_time(refmod, capsys):
    """The reference's scheduler over the full-size bf16 engine (``dropin.bind``: engine log-mel, engine step graph):
    five minutes of long-form audio, 32 slots, word timing off.  With random weights the reference's own stop rules
    end windows after a few dozen tokens and re-encode continuation windows up to twenty times per chunk, and its
    ``decode_batch`` classifies every row on the host at every step, so this is a floor, not a throughput claim:
    the run must finish well ahead of real time.  The measured figure is printed (pytest -s)."""
    import time
    dims = ModelDimensions.from_name("large-v3")
    sd = init_state_dict(dims, 0)
    from whisperdrz.transcriber import Transcriber
    from whisperdrz_b200 import dropin
    from whisperdrz_b200.model import B200Model
    from whisperdrz.tokenizer import get_tokenizer
    model = B200Model(dims, sd, dtype=torch.bfloat16, tokenizer=get_tokenizer(True, num_languages=100, language="en"),
                      max_clips=16)
    t = Transcriber(model_path=None, model=model, lang="en", speaker_remap=False, BS=32, dtw_align=False)
    dropin.bind(t)
    audio = torch.from_numpy(synth.long_form(12, 300.0))
    t.transcribe(audio[: 16000 * 30])                            # warm-up: graphs, tables
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = t.transcribe(audio)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    model.engine.device_status()
    assert len(res.raw_chunks) == 10 and all(r.get("stop_reason") for r in res.raw_chunks)
    windows = sum(1 + (r.get("prediction") or "").count("[CHOP]") for r in res.raw_chunks)
    with capsys.disabled():
        print(f"\n[drop-in, large-v3 bf16, 32 slots] 300 s of audio in {dt:.2f} s = {300.0 / dt:.1f}x real time "
              f"({windows} windows, {sum(t.cuda_graphs.hits.values())} decode steps)")
    assert 300.0 / dt > 10.0
    model.engine.close()


TS = re.compile(r"<\|(\d+\.\d+)\|>")


def test_word_timing_through_the_binding(refmod, small, audio):
    """``dtw_align=True`` (the reference's default): the reference's ``fill_word_timings_batch`` on the CPU
    model against the engine-backed replacement installed by ``dropin.bind``.  The test model has 2 layers
    of 4 heads, so both runs get the same hand-made alignment-head mask instead of the large-v3 one.
    Same text once the timestamps are removed, same number of timestamps, each within one 20 ms frame."""
    dims, sd = small
    mask = torch.zeros(dims.n_text_layer, dims.n_text_head, dtype=torch.bool)
    mask[0, 1] = mask[1, 0] = mask[1, 3] = True
    a = audio[: 16000 * 45]
    tc = _cpu_transcriber(refmod, dims, sd, dtw_align=True)
    tc._dtw_head_mask = mask.clone()
    want = tc.transcribe(a)
    tb = _b200_transcriber(refmod, dims, sd, dtw_align=True)
    tb._dtw_head_mask = mask.clone().to(tb.device)
    got = tb.transcribe(a)
    tb.model.engine.device_status()
    assert TS.sub("", got.text) == TS.sub("", want.text)
    tw, tg = [float(x) for x in TS.findall(want.text)], [float(x) for x in TS.findall(got.text)]
    assert len(tw) == len(tg) and len(tw) > 0
    assert np.abs(np.array(tw) - np.array(tg)).max() <= 0.02 + 1e-9
