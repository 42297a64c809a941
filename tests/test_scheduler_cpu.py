"""Host-only tests of the scheduler, the token-level rules and the multi-rank
sharding, with a stub engine in place of the CUDA library (no GPU)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from whisperdrz_b200 import capi, rules
from whisperdrz_b200.dims import TOK_EOT, TOK_TS_BEGIN
from whisperdrz_b200.sharding import gather_results, shard, split_chunks
from whisperdrz_b200.transcriber import Transcriber, rules_to_array

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class StubEngine:
    """Deterministic stand-in with the Engine methods the scheduler calls.  Its
    "model" proposes tokens from a per-slot counter and obeys the rule
    descriptors the way the device kernel does (forced id, allowed range)."""
    n_slots, max_tokens, max_clips = 4, 448, 2
    device = torch.device("cpu")
    emit_eot = True

    def __init__(self):
        self.calls = {"logmel": 0, "encode": 0, "prefill": 0, "decode": 0}
        self.rows_per_step = []
        self.offsets = []
        self.count = {}

    def device_status(self):
        pass

    def logmel(self, buf, n_samples=None, frame_offset=None):
        self.calls["logmel"] += 1
        self.offsets.append(frame_offset)
        assert buf.shape[0] <= self.max_clips and buf.shape[1] == 480000
        return torch.zeros(buf.shape[0], 128, 3000)

    def encode(self, mel):
        self.calls["encode"] += 1
        return torch.zeros(mel.shape[0], 1500, 8)

    def prefill(self, xa, slots, prompts):
        self.calls["prefill"] += 1
        for s in slots:
            self.count[int(s)] = 0
        return torch.zeros(len(slots), 16)

    def _pick(self, slot, r):
        r = [int(v) for v in r]
        if r[0] >= 0:
            return r[0]
        self.count[slot] += 1
        if r[1] == capi.MODE_ALL_EXCEPT_RANGE:
            if self.emit_eot and r[16] and self.count[slot] % 7 == 0:
                return TOK_EOT                       # cleared id: EOT allowed between pairs
            return min(r[2] + 3, r[3] - 1)
        if r[6] > r[5] and self.count[slot] % 3 == 0:
            return r[6]                              # first allowed closing timestamp
        return 1000 + self.count[slot]               # a text token

    def rules_argmax(self, logits, rules):
        arr = rules.numpy()
        return torch.tensor([self._pick(i, arr[i]) for i in range(len(arr))], dtype=torch.int32)

    def decode_step(self, tokens, slots, rules=None):
        self.calls["decode"] += 1
        self.rows_per_step.append(len(slots))
        arr = rules.numpy()
        return torch.tensor([self._pick(int(s), arr[i]) for i, s in enumerate(slots)], dtype=torch.int32)


def _patch_rules_dev(tr):
    tr._rules_dev = lambda rl: torch.from_numpy(rl if isinstance(rl, np.ndarray) else rules_to_array(rl))


def test_rule_state_machine_pairs_and_budget():
    st = rules.RowState(max_new=5)
    r = st.rule()
    assert r["mode"] == capi.MODE_ALL_EXCEPT_RANGE and r["arg0"] == TOK_TS_BEGIN and r["arg1"] == TOK_TS_BEGIN + 51
    st.update(TOK_TS_BEGIN + 10)                     # opening timestamp
    r = st.rule()
    assert r["table_bits"] == rules.BIT_SPECIAL | rules.BIT_TIMINGS      # a word must follow
    st.update(500)
    r = st.rule()
    assert r["table_bits"] == rules.BIT_SPECIAL and r["prefix_end"] == TOK_TS_BEGIN + 11 and r["pen_ids"] == [500]
    st.update(TOK_TS_BEGIN + 30)                     # closing timestamp
    r = st.rule()
    assert r["mode"] == capi.MODE_ALL_EXCEPT_RANGE and r["arg0"] == TOK_TS_BEGIN + 30 and r["clear_ids"] == [TOK_EOT]
    st.update(TOK_TS_BEGIN + 31)
    st.update(501)
    assert st.rule() == {"forced_id": TOK_EOT}       # budget of 5 reached
    st.update(TOK_EOT)
    assert st.done
    segs = rules.segments(st.tokens, offset=30.0)
    assert segs == [{"start": 30.2, "end": 30.6, "tokens": [500]}]


def test_rules_to_array_layout():
    a = rules_to_array([{"forced_id": 9}, {"mode": 2, "arg0": 5, "arg1": 8, "table_bits": 3, "prefix_begin": 1,
                                         "prefix_end": 4, "set_ids": [7], "clear_ids": [1, 2], "pen_ids": [3, 3, 4]}])
    assert a.shape == (2, 32) and a[0, 0] == 9 and a[1, 0] == -1
    assert list(a[1, 1:7]) == [2, 5, 8, 3, 1, 4]
    assert a[1, 7] == 1 and a[1, 8] == 7 and a[1, 16] == 2 and list(a[1, 17:19]) == [1, 2]
    assert a[1, 21] == 2 and list(a[1, 22:24]) == [3, 4]


def test_scheduler_continuous_batching_with_stub_engine():
    eng = StubEngine()
    tr = Transcriber(eng, max_new_tokens=40, max_continuations=0)
    _patch_rules_dev(tr)
    audio = torch.randn(int(16000 * 30 * 9.5))       # 10 chunks for 4 slots
    res = tr.transcribe(audio)
    assert [r["id"] for r in res.raw_chunks] == [f"chunk_{i}" for i in range(10)]
    assert res.raw_chunks[-1]["duration"] == pytest.approx(15.0)
    assert all(r["stop_reason"] in ("eot", "max_tokens") for r in res.raw_chunks)
    assert all(s.status == "ready" for s in tr.states) and not tr.pending_chunks
    # slots are refilled as they finish: some steps run with fewer than 4 rows only at the tail
    assert max(eng.rows_per_step) == 4 and eng.calls["prefill"] >= 3
    # offsets are applied to the segments of later chunks
    assert res.raw_chunks[3]["segments"][0]["start"] >= 90.0
    assert abs(tr.seconds_processed - 285.0) < 1e-6
    # timestamps inside a chunk never go backwards
    for r in res.raw_chunks:
        ts = [t for t in r["tokens"] if t >= TOK_TS_BEGIN]
        assert ts == sorted(ts)


def test_pipeline_call_and_flush():
    eng = StubEngine()
    tr = Transcriber(eng, max_new_tokens=12)
    _patch_rules_dev(tr)
    chunks = split_chunks(torch.randn(16000 * 70))
    assert [c["duration"] for c in chunks] == [30.0, 30.0, 10.0]
    assert tr(chunks[0]) is None                     # buffering: fewer chunks than free slots
    out = list(tr.flush())
    assert len(out) == 1 and out[0]["id"] == "chunk_0"
    tr(chunks[1:])
    assert {r["id"] for r in tr.flush()} == {"chunk_1", "chunk_2"}


def test_sharding_is_a_partition():
    chunks = [{"id": f"chunk_{i}"} for i in range(11)]
    parts = [shard(chunks, r, 4) for r in range(4)]
    assert sorted(c["id"] for p in parts for c in p) == sorted(c["id"] for c in chunks)
    assert [len(p) for p in parts] == [3, 3, 3, 2]
    assert gather_results(list(reversed(chunks)), 0, 1) == chunks


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
from test_scheduler_cpu import AlignStubEngine, _patch_rules_dev
from whisperdrz_b200.alignment import token_aligner
from whisperdrz_b200.transcriber import Transcriber
from whisperdrz_b200.sharding import transcribe_sharded
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
tr = Transcriber(AlignStubEngine(), max_new_tokens=20, aligner=token_aligner); _patch_rules_dev(tr)
torch.manual_seed(0)
audio = torch.randn(16000 * 30 * 7)
res = transcribe_sharded(tr, audio, rank, world)
if rank == 0:
    assert [r["id"] for r in res.raw_chunks] == [f"chunk_{i}" for i in range(7)], res.raw_chunks
    assert all(len(r["word_times"]) >= 1 for r in res.raw_chunks)      # word timing travels with the gathered chunks
    print("GATHERED", len(res.raw_chunks), len(res.segments))
else:
    assert res is None
dist.destroy_process_group()
"""


def test_two_rank_sharding_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29731")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29731", str(script), ROOT]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "GATHERED 7" in out.stdout


def test_batch_rule_state_equals_row_state():
    """The vectorised state used by the scheduler and the per-row reference
    implementation give the same descriptors and the same bookkeeping on random
    token streams that follow the rules."""
    rng = np.random.default_rng(0)
    n = 16
    rows = [rules.RowState(max_new=30) for _ in range(n)]
    bs = rules.BatchRuleState(n, 30)
    for _ in range(40):
        act = [i for i in range(n) if not rows[i].done]
        if not act:
            break
        a = rules_to_array([rows[i].rule() for i in act])
        b = bs.rules_array(act)
        for r in range(len(act)):
            ra, rb = a[r].copy(), b[r].copy()
            assert set(ra[22: 22 + ra[21]]) == set(rb[22: 22 + rb[21]])   # penalty ids as sets
            ra[21:] = 0
            rb[21:] = 0
            assert (ra == rb).all(), (ra, rb)
        toks = []
        for r in a:
            if r[0] >= 0:
                t = int(r[0])
            elif r[1] == capi.MODE_ALL_EXCEPT_RANGE:
                t = TOK_EOT if (r[16] and rng.random() < 0.1) else int(rng.integers(r[2], r[3]))
            elif r[6] > r[5] and r[6] < 51866 and rng.random() < 0.4:
                t = int(rng.integers(r[6], 51866))           # a closing timestamp after the opening one
            else:
                t = int(rng.integers(0, 50000))
            toks.append(t)
        for i, t in zip(act, toks):
            rows[i].update(t)
        done = bs.update(act, toks)
        assert list(done) == [rows[i].done for i in act]
    assert all(r.done for r in rows)
    for i in range(n):
        assert bs.slot_tokens(i) == rows[i].tokens


def test_continuation_windows_restart_at_the_last_closing_timestamp():
    """A window that hits its token budget before the end of its chunk is
    continued from its last closing timestamp (reference: transcriber.py:1283-1334):
    the kept tokens end on a closing timestamp, the next window's mel starts at
    that offset, segments stay monotonic, and the cap on continuations holds."""
    eng = StubEngine()
    eng.emit_eot = False                              # windows end only by running out of tokens
    tr = Transcriber(eng, max_new_tokens=12, max_continuations=3)
    _patch_rules_dev(tr)
    res = tr.transcribe(torch.randn(16000 * 30))
    r = res.raw_chunks[0]
    assert r["windows"] == 4 and r["stop_reason"] == "max_tokens"       # 1 + 3 continuations, then emitted
    offs = [o[0] for o in eng.offsets if o is not None]
    assert len(offs) == 3 and offs == sorted(offs) and offs[0] >= 100   # each window starts >= 1 s later
    starts = [s["start"] for s in r["segments"]]
    assert starts == sorted(starts) and all(s["end"] > s["start"] for s in r["segments"])
    # every kept window contributes an even number of timestamps (closed pairs only)
    n_ts = sum(1 for t in r["tokens"] if t >= TOK_TS_BEGIN)
    assert n_ts >= 2 * len(r["segments"]) - 1
    eng0 = StubEngine()
    eng0.emit_eot = False
    tr0 = Transcriber(eng0, max_new_tokens=12, max_continuations=0)
    _patch_rules_dev(tr0)
    assert tr0.transcribe(torch.randn(16000 * 30)).raw_chunks[0]["windows"] == 1


class AlignStubEngine(StubEngine):
    """Adds the alignment calls: the 'matrix' makes the cheapest path a straight diagonal, and the DTW is
    the oracle's, so the scheduler's bookkeeping (which tokens are words, window offsets, what a continuation
    keeps) is what gets tested."""
    dims = type("D", (), {"n_audio_ctx": 1500})()

    def __init__(self):
        super().__init__()
        self.align_calls = []
        self.heads = None

    def align_configure(self, heads):
        self.heads = list(heads)

    def align_matrix(self, tokens, lens, slots, caps):
        self.align_calls.append((np.asarray(tokens).copy(), list(lens), list(slots), list(caps)))
        B, T = np.asarray(tokens).shape
        m = torch.zeros(B, T, 1500)
        for b in range(B):
            for t in range(lens[b]):
                m[b, t, min(1499, 10 * t)] = 5.0          # high attention = low cost along a diagonal
        return m

    def dtw(self, matrix, row0, n_rows, n_cols, limits=None):
        from oracle import oracle
        out = []
        for b in range(matrix.shape[0]):
            x = -matrix[b, row0[b]: row0[b] + n_rows[b], : n_cols[b]].numpy()
            if limits is not None:
                lo, hi = limits[b]
                cols = np.arange(x.shape[1])[None, :]
                x = np.where((cols < lo[:, None]) | (cols >= hi[:, None]), np.inf, x)
            out.append(oracle.dtw_path(x))
        return out


def test_finished_windows_are_aligned_before_their_slot_is_reused():
    from whisperdrz_b200 import alignment
    eng = AlignStubEngine()
    tr = Transcriber(eng, max_new_tokens=40, max_continuations=0, aligner=alignment.token_aligner)
    _patch_rules_dev(tr)
    res = tr.transcribe(torch.randn(16000 * 70))              # three chunks over two prefill batches of the 4-slot stub
    assert eng.heads == alignment.ALIGNMENT_HEADS_LARGE_V3 and tr.windows_aligned == len(res.raw_chunks) == 3
    for r in res.raw_chunks:
        words = r["word_times"]
        text_pos = [i for i, t in enumerate(r["tokens"]) if t < TOK_EOT]
        assert [w[0] for w in words] == text_pos               # every text token is a word, in order
        starts = [w[1] for w in words]
        assert starts == sorted(starts) and all(w[2] >= w[1] for w in words)
        assert starts[0] >= r["offset"] and words[-1][2] <= r["offset"] + 30.0 + 1e-6
    # the pass saw sot + lang + transcribe + no-timestamps + the text tokens + eot, in the chunk's own slot
    toks, lens, slots, caps = eng.align_calls[0]
    assert toks[0, :4].tolist() == [50258, 50259, 50360, 50364] and toks[0, lens[0] - 1] == TOK_EOT
    assert all(0 <= s < eng.n_slots for s in slots) and caps[0] == 1500


def test_continuation_keeps_the_words_of_the_kept_tokens():
    from whisperdrz_b200 import alignment
    eng = AlignStubEngine()
    eng.emit_eot = False
    tr = Transcriber(eng, max_new_tokens=12, max_continuations=2, aligner=alignment.token_aligner)
    _patch_rules_dev(tr)
    r = tr.transcribe(torch.randn(16000 * 30)).raw_chunks[0]
    assert r["windows"] == 3 and tr.windows_aligned == 3
    idx = [w[0] for w in r["word_times"]]
    assert idx == sorted(idx) and len(set(idx)) == len(idx)
    assert all(r["tokens"][i] < TOK_EOT for i in idx)            # indices point at text tokens of the stitched chunk
    assert len(idx) >= 3 and all(w[2] >= w[1] >= 0.0 for w in r["word_times"])


def test_warm_slots_are_prefilled_in_the_background_and_promoted():
    """n_warm extra slots (transcriber.py:559-568, 976-1040): the same chunks give the same tokens as the
    plain scheduler, at most BS slots decode at a time, and slots enter decoding through the warm pool."""
    audio = torch.randn(16000 * 30 * 9)
    tp = Transcriber(StubEngine(), BS=2, max_new_tokens=12, max_continuations=0)
    _patch_rules_dev(tp)
    plain = tp.transcribe(audio)
    eng = StubEngine()
    t = Transcriber(eng, BS=2, n_warm=2, max_new_tokens=12, max_continuations=0)
    _patch_rules_dev(t)
    warm = t.transcribe(audio)
    assert [r["id"] for r in warm.raw_chunks] == [r["id"] for r in plain.raw_chunks] == [f"chunk_{i}" for i in range(9)]
    assert all(r["stop_reason"] in ("eot", "max_tokens") and r["tokens"] for r in warm.raw_chunks)
    assert all(s.status == "ready" for s in t.states) and not t.pending_chunks
    assert max(eng.rows_per_step) <= 2
    assert t.promoted == 9 and not t.warming
    with pytest.raises(ValueError):
        Transcriber(StubEngine(), BS=4, n_warm=1)
