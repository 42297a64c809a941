"""Timings of the named workloads other than the batched end-to-end case that
bench.py times, on one GPU:

    python bench_configs.py [cfg1 cfg2 cfg3 cfg5 cfg5w cfg5b cfg5_small align align_small products products_once]

cfg1  one 30 s clip, 4-token prompt, 224 greedy tokens with EOS suppressed (latency; fp32 and bf16)
cfg2  encoder only, bf16, 16 clips: log-mel + conv stem + 32 layers (time, TFLOP/s)
cfg3  batched decode, bf16: 32 slots over precomputed cross K/V, prompts U{4..64}, generated U{32..448},
      forced EOS at the drawn length, timestamp-pair rules (tokens/s)
cfg5  serving: 1024 requests with log-uniform durations 5 s - 10 min and Poisson arrivals offered faster than one
      GPU drains them, chunks of different requests packed into shared decode steps (throughput, p50/p99 time
      to final transcript); ``cfg5w``: 32 of the 256 slots as a warm pool prefilled on a side stream;
      ``cfg5b``: refill in groups of 8; ``cfg5_small``: 96 requests
cfg4  (in bench.py: key ``cfg4_strong_rtfx``) one hour of long-form audio, 120 chunks sharded over the ranks
align word-timing alignment of 8 finished windows, 445 tokens each (the longest a chunk gets), bf16: the
      teacher-forced pass + scores + cost matrix, and the DTW with its download (``align_small``: 155 tokens,
      the size a 224-token window gives at token level)
products  the decode step's weight products (wdz_linear_rows) at 32 and 256 token rows, each shape replayed
      inside a CUDA graph over a 300 MB rotation of weights (so they stream from HBM as in a decode step)

Inputs are the seeded synthetic stand-ins of ``synth``; weights are seeded random init.  Prints one JSON
object per workload."""
from __future__ import annotations

import json
import sys
import time

import numpy as np
import torch

import os

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from whisperdrz_b200 import capi, synth  # noqa: E402
from whisperdrz_b200.dims import ModelDimensions, TOK_EOT  # noqa: E402
from whisperdrz_b200.engine import Engine  # noqa: E402
from whisperdrz_b200.rules import timestamp_tables  # noqa: E402
from whisperdrz_b200.transcriber import Transcriber  # noqa: E402
from whisperdrz_b200.weights import init_state_dict  # noqa: E402

ENC_GFLOP_PER_CLIP = 2274.0  # conv 17.7 + 32 x (59.0 GEMM + 11.5 attention)


def _timed(fn, reps=3, warm=1):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        out = fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps, out


def cfg1(dims, sd):
    res = {"workload": "cfg1: 1 clip, prompt [sot, en, transcribe, <0.00>], 224 greedy tokens, EOS suppressed"}
    audio = torch.from_numpy(synth.clips([1])).cuda()
    for name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        e = Engine(dims, sd, dtype=dt, n_slots=2, max_clips=1)
        rule = e.rules_to_device([{"set_ids": [TOK_EOT]}])

        def run():
            xa = e.encode(e.logmel(audio))
            cur = e.rules_argmax(e.prefill(xa, [0], [[50258, 50259, 50360, 50365]]), rule)
            toks = [cur]
            for _ in range(223):
                cur = e.decode_step(cur, [0], rules=rule)
                toks.append(cur)
            return torch.cat(toks).tolist()
        ms, toks = _timed(run, reps=2)
        res[name] = {"latency_ms": ms, "rtfx": 30000.0 / ms, "tokens": len(toks)}
        if dt == torch.bfloat16:
            # the same decode with the rule state on the device: all 223 steps queued by one call
            def run_dev():
                xa = e.encode(e.logmel(audio))
                logits = e.prefill(xa, [0], [[50258, 50259, 50360, 50365]])
                e.ts_reset([0], [224])
                e.ts_first(logits, [0])
                e.ts_steps([0], 223)
                return e.ts_tokens(0, int(e.ts_poll()[0, 1]))
            ms2, toks2 = _timed(run_dev, reps=2)
            res["bf16_device_rules"] = {"latency_ms": ms2, "rtfx": 30000.0 / ms2, "tokens": len(toks2)}
        e.close()
    return res


def cfg2(dims, sd, flags=0):
    e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=2, max_clips=16, flags=flags)
    audio = torch.from_numpy(synth.clips(range(1, 17))).cuda()
    ms_mel, mel = _timed(lambda: e.logmel(audio))
    ms_enc, _ = _timed(lambda: e.encode(mel))
    e.close()
    return {"workload": "cfg2: encoder only, bf16, 16 clips", "logmel_ms": ms_mel, "encoder_ms": ms_enc,
            "encoder_tflops": 16 * ENC_GFLOP_PER_CLIP / ms_enc, "rtfx_encoder_only": 16 * 30000.0 / (ms_mel + ms_enc)}


def cfg3(dims, sd):
    B = 32
    e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=B, max_clips=16, max_rows=2048,
               tables=timestamp_tables(dims.n_vocab))
    audio = torch.from_numpy(synth.clips(range(1, B + 1))).cuda()
    for i in range(0, B, 16):
        e.cross_kv(e.encode(e.logmel(audio[i: i + 16])), list(range(i, i + 16)))
    p_len, g_len, prompts = synth.decode_lengths(2, B, dims.n_text_ctx)

    def run():
        # rule state on the device: eight decode steps per host round trip, rows that reach their drawn length are
        # forced to EOS and dropped there; the host only re-stages the list of live slots between polls
        e.slot_reset(range(B))
        tok, sl, pos, emit = [], [], [], []
        for b in range(B):
            for j, t in enumerate(prompts[b]):
                tok.append(int(t)); sl.append(b); pos.append(j)
            emit.append(len(tok) - 1)
        logits = e.forward_rows(tok, sl, pos, emit_rows=emit)
        ids = list(range(B))
        e.ts_reset(ids, [int(g) for g in g_len])
        e.ts_first(logits, ids)
        steps = 0
        while ids:
            e.ts_steps(ids, 8)
            steps += 8
            st = e.ts_poll()
            ids = [i for i in ids if not st[i][6]]
        n_tok = int(e.ts_poll()[:B, 1].sum())
        return n_tok, steps
    ms, (n_tok, steps) = _timed(run, reps=2)
    e.close()
    return {"workload": "cfg3: 32 slots, ragged prompts 4-64 and lengths 32-448, forced EOS, timestamp-pair rules",
            "ms": ms, "tokens": n_tok, "decode_steps": steps, "tokens_per_s": n_tok / ms * 1e3,
            "prompt_rows": int(p_len.sum()), "mean_generated": float(g_len.mean())}


def cfg5(dims, sd, n_req=1024, slots=256, seed=4, min_refill=1, n_warm=0, offered=2500.0):
    e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=slots, max_clips=16, tables=timestamp_tables(dims.n_vocab))
    tr = Transcriber(e, max_new_tokens=224, max_continuations=0, min_refill=min_refill, n_warm=n_warm)
    dur = synth.request_durations(seed, n_req)
    total_audio = float(dur.sum())
    rate = offered / float(dur.mean())          # offered load above what one GPU sustains: keeps it saturated
    arrive = synth.poisson_arrivals(seed, n_req, rate)
    base = synth.long_form(3, 630.0)            # every request is a window of one synthetic recording
    left, final = {}, {}
    nxt, t0 = 0, time.perf_counter()
    while len(final) < n_req:
        now = time.perf_counter() - t0
        while nxt < n_req and arrive[nxt] <= now:
            n = int(dur[nxt] * 16000)
            a = torch.from_numpy(base[:n])
            parts = [a[c: c + 480000] for c in range(0, n, 480000)]
            parts = [p for i, p in enumerate(parts) if i == 0 or len(p) >= 1600]   # drop a sub-0.1 s tail
            left[nxt] = len(parts)
            for c, part in enumerate(parts):
                tr.pending_chunks.append({"audio": part, "id": f"r{nxt}_{c}", "duration": len(part) / 16000,
                                          "offset": 30.0 * c, "req": nxt})
            nxt += 1
        if not tr.busy():
            time.sleep(max(0.0, min(0.005, arrive[nxt] - now)))
            continue
        for res in tr.step():
            r = res["req"]
            left[r] -= 1
            if left[r] == 0:
                final[r] = time.perf_counter() - t0 - arrive[r]
    wall = time.perf_counter() - t0
    lat = np.array(sorted(final.values()))
    e.close()
    return {"workload": f"cfg5: {n_req} requests, durations log-uniform 5 s-10 min, Poisson arrivals, {slots} slots "
                        f"({n_warm} of them warm), min_refill {min_refill}",
            "audio_s": total_audio, "wall_s": wall, "rtfx": total_audio / wall, "offered_rtfx": offered,
            "p50_s": float(lat[len(lat) // 2]), "p99_s": float(lat[min(len(lat) - 1, int(0.99 * len(lat)))]),
            "decode_steps": tr.steps, "mean_rows_per_step": tr.launch_rows / max(tr.steps, 1)}


def align(dims, sd, n_chunks=8, n_ids=440, reps=3):
    from whisperdrz_b200 import alignment as A
    e = Engine(dims, sd, dtype=torch.bfloat16, n_slots=n_chunks, max_clips=8, max_rows=4096)
    g = torch.Generator(device="cpu").manual_seed(6)
    xa = (torch.randn(n_chunks, dims.n_audio_ctx, dims.n_audio_state, generator=g) * 0.5).to(torch.bfloat16).cuda()
    slots = list(range(n_chunks))
    e.cross_kv(xa, slots)
    e.align_configure(A.ALIGNMENT_HEADS_LARGE_V3)
    rng = np.random.RandomState(0)
    tokens, lens = A.build_full_tokens([rng.randint(0, 50000, size=n_ids).tolist() for _ in range(n_chunks)])
    caps = [dims.n_audio_ctx] * n_chunks
    ms_matrix, m = _timed(lambda: e.align_matrix(tokens, lens, slots, caps), reps=reps)
    ms_dtw, paths = _timed(lambda: e.dtw(m, [3] * n_chunks, [ln - 4 for ln in lens], caps), reps=reps)
    e.device_status()
    rows = n_chunks * tokens.shape[1]
    n_layers = max(l for l, _ in A.ALIGNMENT_HEADS_LARGE_V3) + 1
    d = dims.n_text_state
    gflop = rows * n_layers * 2.0 * (12 * d * d) / 1e9            # the pass's products (attention not counted)
    out = {"workload": f"align: {n_chunks} windows x {tokens.shape[1]} tokens, bf16, alignment heads of large-v3",
           "matrix_ms": ms_matrix, "dtw_ms": ms_dtw, "ms_per_window": (ms_matrix + ms_dtw) / n_chunks,
           "pass_gemm_tflops": gflop / ms_matrix, "path_len": int(len(paths[0][0]))}
    e.close()
    return out


def products(dims, sd, row_counts=(32, 256, 384), once=False):
    """``once``: every shape launched a single time outside a graph, on cold weights (for profiler captures)."""
    small = ModelDimensions.from_name("test-small")
    e = Engine(small, init_state_dict(small, 0), dtype=torch.bfloat16, n_slots=2, max_clips=1)
    d = dims.n_text_state
    shapes = {"qkv": (3 * d, d), "attn_out / cross_out (residual)": (d, d), "cross_q": (d, d), "fc1": (4 * d, d),
              "fc2 (residual)": (d, 4 * d)}
    g = torch.Generator(device="cpu").manual_seed(8)
    out = {"workload": "decode products in a CUDA graph, weights rotated through 300 MB", "us": {}}
    for name, (N, K) in shapes.items():
        nw = max(2, int(300e6 / (N * K * 2)))
        ws = [(torch.randn(N, K, generator=g) * 0.03).to(torch.bfloat16).cuda() for _ in range(nw)]
        for M in row_counts:
            x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
            acc = torch.zeros(M, N, device="cuda") if "residual" in name else None
            if once:
                ms, _ = _timed(lambda: e.linear_rows(x, ws[1], out=acc), reps=1, warm=0)
                out["us"][f"{name} N{N} K{K} rows{M}"] = round(ms * 1e3, 2)
                continue
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                e.linear_rows(x, ws[0], out=acc)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(nw):
                    e.linear_rows(x, ws[i], out=acc)
            ms, _ = _timed(graph.replay, reps=5, warm=2)
            out["us"][f"{name} N{N} K{K} rows{M}"] = round(ms * 1e3 / nw, 2)
        del ws
    e.close()
    return out


def enc_products(dims, sd, rows=48000, once=False):
    """The encoder's four products on their own (bias, bf16 out; fc1 with and without its GELU), CTA pairs against
    lone CTAs.  ``once``: the fc1 + GELU product launched a single time per kernel (for profiler captures)."""
    small = ModelDimensions.from_name("test-small")
    e = Engine(small, init_state_dict(small, 0), dtype=torch.bfloat16, n_slots=2, max_clips=1)
    d = dims.n_audio_state
    shapes = {"qkv": (3 * d, d, False), "out": (d, d, False), "fc1 + gelu": (4 * d, d, True),
              "fc1 without gelu": (4 * d, d, False), "fc2": (d, 4 * d, False)}
    if once:
        shapes = {"fc1 + gelu": shapes["fc1 + gelu"]}
    g = torch.Generator(device="cpu").manual_seed(9)
    out = {"workload": f"encoder products, {rows} rows, bf16", "us_tflops": {}}
    for name, (N, K, gelu) in shapes.items():
        x = torch.randn(rows, K, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(N, K, generator=g) * 0.03).to(torch.bfloat16).cuda()
        b = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
        for mode, label in ((0, "pairs"), (2, "lone")):
            ms, _ = _timed(lambda: e.linear(x, w, b, gelu=gelu, cuda_cores_only=mode), reps=1 if once else 20,
                           warm=0 if once else 3)
            out["us_tflops"][f"{name} N{N} K{K} {label}"] = [round(ms * 1e3, 1), round(2.0 * rows * N * K / ms / 1e9, 1)]
    e.close()
    return out


def main(argv):
    want = argv or ["cfg1", "cfg2", "cfg3", "cfg5"]
    dims = ModelDimensions.from_name("large-v3")
    sd = init_state_dict(dims, 0)
    fns = {"cfg1": cfg1, "cfg2": cfg2, "cfg3": cfg3, "cfg5": cfg5,
           "cfg2_lone_cta": lambda d, s: cfg2(d, s, flags=capi.FLAG_NO_CTA_PAIRS),
           "cfg5b": lambda d, s: cfg5(d, s, min_refill=8), "cfg5w": lambda d, s: cfg5(d, s, n_warm=32),
           "cfg5_small": lambda d, s: cfg5(d, s, n_req=96, offered=1500.0), "align": align,
           "align_small": lambda d, s: align(d, s, n_ids=150), "products": products,
           "products_once": lambda d, s: products(d, s, row_counts=(256,), once=True),
           "enc_products": enc_products,
           "enc_products_once": lambda d, s: enc_products(d, s, rows=24000, once=True)}
    with torch.inference_mode():
        for w in want:
            print(json.dumps(fns[w](dims, sd)), flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
