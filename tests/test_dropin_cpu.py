"""Host logic of the drop-in binding (whisperdrz_b200/dropin.py) without a GPU: the log-mel stand-in, the step-graph
stand-in, the slot lookup, and the word-timing replacement with the engine's alignment faked (the reference's own text
functions come from oracle/_ref)."""
import pytest
import torch

from oracle import ref
from whisperdrz_b200 import dropin
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.model import B200Model


class _FakeEngine:
    max_clips, device = 2, torch.device("cpu")
    align_heads = None

    def __init__(self):
        self.calls = []

    def logmel(self, audio):
        self.calls.append(tuple(audio.shape))
        B = audio.shape[0]
        return torch.arange(3000, dtype=torch.float32).repeat(B, 4, 1)

    def align_configure(self, heads):
        self.align_heads = [tuple(h) for h in heads]


def _model():
    m = B200Model(ModelDimensions.from_name("test-tiny"), {}, dtype=torch.float32, device="cpu", tokenizer=object())
    m.engine = _FakeEngine()
    return m


def test_engine_logmel_shapes_padding_and_fallback():
    m = _model()
    host_calls = []
    host = lambda audio, target_frames=None: host_calls.append((tuple(audio.shape), target_frames)) or "host"
    tomel = dropin.EngineLogMel(m, host)
    out = tomel(torch.zeros(3, 16000 * 10))                       # three clips of 10 s: two engine calls (max_clips 2)
    assert out.shape == (3, 4, 1000) and m.engine.calls == [(2, 160000), (1, 160000)]
    assert torch.equal(out[0, 0], torch.arange(1000, dtype=torch.float32))
    one = tomel(torch.zeros(16000 * 7), target_frames=3000)       # 1-D in, 2-D out, padded with -1.5
    assert one.shape == (4, 3000) and float(one[0, 699]) == 699.0 and float(one[0, 700]) == -1.5
    assert tomel(torch.zeros(1, 480001)) == "host" and tomel(torch.zeros(1, 399), target_frames=5) == "host"
    assert host_calls == [((1, 480001), None), ((1, 399), 5)]


def test_slot_lookup_from_a_cache_row():
    cache = torch.zeros(5, 1500, 8)
    assert dropin._slot_of(cache[3], cache) == 3
    assert dropin._slot_of(cache[0], cache) == 0
    with pytest.raises(ValueError):
        dropin._slot_of(torch.zeros(1500, 8), cache)


def test_step_graphs_forward_goes_through_the_model():
    m = _model()
    seen = {}

    class Dec:
        def forward_flash(self, tokens, skv, ckv, positions, slot_indices=None, return_hidden_states=False):
            seen["args"] = (tokens.shape, positions.tolist(), slot_indices.tolist())
            return "logits"
    m.decoder = Dec()
    g = dropin.EngineStepGraphs(m)
    assert g.forward(torch.zeros(3, 1, dtype=torch.long), torch.tensor([4, 5, 6]), torch.tensor([0, 2, 1])) == "logits"
    assert seen["args"] == (torch.Size([3, 1]), [4, 5, 6], [0, 2, 1]) and g.hits[3] == 1


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref is not installed")
def test_word_timing_replacement_rebuilds_text_like_the_reference(monkeypatch):
    """With the engine's alignment replaced by fixed word times, the replacement must write them into the text
    exactly as the reference's own rebuild does, and calls for other model objects must reach the original."""
    ref.load()
    import whisperdrz.dtw_align as D
    from whisperdrz.tokenizer import get_tokenizer
    tok = get_tokenizer(True, num_languages=100, language="en")
    m = _model()
    xa_cache = torch.zeros(4, 1500, 8)
    text = "[0] <|0.50|>hello<|0.90|> there my friend\n[1] <|2.00|>yes<|2.40|> indeed"
    seen = {}

    def fake_align(engine, chunks, sot_sequence=None, no_timestamps=None, eot=None):
        seen["chunks"] = chunks
        return [[(0.1 * i, 0.1 * i + 0.05) for i in range(len(c.word_lens))] for c in chunks]
    monkeypatch.setattr(dropin.alignment, "align_chunks", fake_align)
    original = lambda *a, **k: "original"
    fn = dropin.make_fill_word_timings_batch(D, original, lambda model: xa_cache)
    mask = torch.zeros(2, 2, dtype=torch.bool)
    mask[1, 0] = True
    out = fn(m, tok, [(xa_cache[2], text, 3000), (xa_cache[1], "", 3000)], head_mask=mask)
    assert m.engine.align_heads == [(1, 0)]
    ch = seen["chunks"]
    assert len(ch) == 1 and ch[0].slot == 2 and ch[0].num_frames == 3000
    assert sum(ch[0].word_lens) == len(ch[0].ids) and (1, 0.5, 0.9) in [tuple(a) for a in ch[0].word_anchors]
    # what the reference's own rebuild gives for the same word times
    lines, flat, tags = D.parse_predicted_lines(text)
    rec = D._prepare_chunk(D.chunk_speaker_lines(lines, tok, 440)[0], tok, flat, tags, 440)
    times = [None] * len(flat)
    for i, (oi, _) in enumerate(rec["tagged"]):
        if oi is not None:
            times[oi] = (0.1 * i, 0.1 * i + 0.05)
    assert out == [D.rebuild_with_timings(text, flat, times), ""]
    assert out[0].count("<|") > text.count("<|")                   # the untimed words got timestamps
    assert fn(object(), tok, [(xa_cache[0], text, 3000)]) == "original"
