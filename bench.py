#!/usr/bin/env python
"""Throughput of the transcription hot path on B200.

One step = one pass of the whole path over a batch of 30 s synthetic chunks on
each GPU: log-mel -> large-v3 encoder -> cross K/V + prompt prefill -> greedy
decode of --new-tokens tokens per chunk under the timestamp-pair logit rules,
driven by the continuous-batching scheduler.  Metric: audio seconds per wall
second (RTFx), whole job over all ranks.

  value : audio already resident in HBM when the timed region starts
  e2e   : the same through the public API with pinned HOST audio (H2D inside)
  roofline : the decode cross-attention kernel (the dominant byte mover),
             timed with CUDA events inside the engine on one extra step
  cpu_baseline : the reference's CPU classes on a bounded sample, rank 0, N=1 only

``--impl reference`` times the reference's own CPU implementation of the path
(its unmodified classes, installed into oracle/_ref by oracle/make_ref.py; the
oracle port only when that install is absent) on the host cores, one bounded
sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "audio-sec/sec (RTFx)"
UNIT = "audio-s/s"
PROMPT = [50258, 50259, 50360]


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks / throttle reasons of one GPU while running."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [x.strip() for x in out.stdout.strip().split(",")]
                if len(parts) >= 6:
                    self.rows.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self) -> dict:
        self.stop_flag.set()
        self.join(timeout=6)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = sorted(float(r[0]) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
REF_BATCH = 8      # the CPU arm decodes this many chunks per step
REF_CYCLE = 4      # and spreads one chunk's share of a pass over this many bench steps


class CpuArm:
    """The reference's own classes (unmodified, from oracle/_ref: ``LogMelSpectrogram``, ``model.encoder``,
    ``prefill_flash``, ``decoder.forward_flash`` through its SDPA path) on the host cores, in fp32.

    The unit of work is 1/REF_BATCH of a pass over REF_BATCH chunks (= 30 s of audio): log-mel + encoder +
    cross K/V + prompt of ONE chunk, and new_tokens / REF_BATCH decode steps over REF_BATCH rows whose cache
    depths are spread evenly over the new_tokens positions.  Greedy arg-max, no logit rules (their cost is
    host string work in the reference).  A unit takes about half a minute of CPU, so it is cut into
    REF_CYCLE bench steps: every step runs 1/REF_CYCLE of the unit's decode steps and every REF_CYCLE-th
    step also the encoder side.  Without oracle/_ref the CPU port (oracle/oracle.py) runs the same work."""

    def __init__(self, sd, dims, new_tokens: int):
        from oracle import ref
        from whisperdrz_b200 import synth
        self.dims, self.new_tokens = dims, new_tokens
        self.n_decode = max(REF_CYCLE, new_tokens // REF_BATCH)          # decode steps of one unit
        self.per_step = max(1, self.n_decode // REF_CYCLE)
        self.audio = torch.from_numpy(synth.clip(1))
        self.depths = [len(PROMPT) + int((j + 0.5) * new_tokens / self.n_decode) for j in range(self.n_decode)]
        self.cursor = 0
        self.tok = torch.full((REF_BATCH, 1), 1000, dtype=torch.long)
        self.model = ref.model(dims, sd)
        if self.model is not None:
            from whisperdrz.audio import LogMelSpectrogram
            self.kind = "reference"
            self.tomel = LogMelSpectrogram(dims.n_mels)
            self.model.decoder.cache_embedding_weight(torch.float32)
            self.self_kv, self.cross_kv = self.model.create_flash_kv(REF_BATCH, max_tokens=dims.n_text_ctx)
        else:
            from oracle import oracle
            self.kind = "port"
            self.oracle = oracle
            self.dec = oracle.SlotDecoder(sd, dims.n_text_layer, dims.n_text_head, REF_BATCH, dims.n_text_ctx)
            self.sd = sd

    def describe(self, timed_decode_steps: int, encoder_passes: int) -> str:
        return (f"unit = 1/{REF_BATCH} of a pass over {REF_BATCH} chunks (30 s of audio): log-mel + encoder + cross K/V + "
                f"prompt of 1 chunk, {self.n_decode} decode steps over {REF_BATCH} rows at cache depths spread over the "
                f"{self.new_tokens} positions; greedy, no logit rules. Timed here: {encoder_passes} encoder-side pass(es) "
                f"and {timed_decode_steps} decode steps; seconds per unit = mean encoder-side time + {self.n_decode} x "
                f"mean decode-step time")

    @torch.inference_mode()
    def encoder_side(self) -> float:
        t0 = time.perf_counter()
        if self.kind == "reference":
            m = self.model
            xa = m.encoder(self.tomel(self.audio[None], target_frames=3000))
            m.prefill_flash(torch.tensor([PROMPT]), xa, self.self_kv, self.cross_kv, torch.tensor([0]))
        else:
            o = self.oracle
            mel = o.window_mel(o.log_mel(self.audio))[None]
            xa = o.encoder(self.sd, mel, self.dims.n_audio_layer, self.dims.n_audio_head)
            self.dec.prefill(torch.tensor([PROMPT]), xa, [0])
        return time.perf_counter() - t0

    @torch.inference_mode()
    def decode_steps(self, n: int) -> float:
        slots = torch.arange(REF_BATCH)
        t0 = time.perf_counter()
        for _ in range(n):
            depth = self.depths[self.cursor % len(self.depths)]
            self.cursor += 1
            if self.kind == "reference":
                for kv in self.self_kv:
                    kv.seq_lens[:] = depth
                pos = self.self_kv[0].seq_lens[slots]
                logits = self.model.decoder.forward_flash(self.tok, self.self_kv, self.cross_kv, pos,
                                                          slot_indices=slots)
            else:
                self.dec.seq_lens[:] = depth
                logits = self.dec.forward(self.tok, list(range(REF_BATCH)))
            self.tok = logits[:, -1].argmax(-1, keepdim=True)
        return time.perf_counter() - t0

    def seconds_per_unit(self, enc_times, dec_time: float, dec_steps: int) -> float:
        return float(np.mean(enc_times)) + self.n_decode * dec_time / max(dec_steps, 1)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from whisperdrz_b200.dims import ModelDimensions
    from whisperdrz_b200.weights import init_state_dict
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dims = ModelDimensions.from_name(args.model)
    arm = CpuArm(init_state_dict(dims, 0), dims, args.new_tokens)
    enc_all, enc_timed, dec_time, dec_steps, wall = [], [], 0.0, 0, 0.0
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        if i % REF_CYCLE == 0:
            enc_all.append(arm.encoder_side())
            if i >= args.warmup:
                enc_timed.append(enc_all[-1])
        d = arm.decode_steps(arm.per_step)
        if i >= args.warmup:
            dec_time += d
            dec_steps += arm.per_step
            wall += time.perf_counter() - t0
    per_unit = arm.seconds_per_unit(enc_timed or enc_all, dec_time, dec_steps)
    v = 30.0 / per_unit
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / max(args.steps, 1) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": arm.kind,
                             "sample": arm.describe(dec_steps, len(enc_timed or enc_all)),
                             "seconds_per_30s_chunk": per_unit},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args) -> dict:
    return {"workload": f"batched 30 s chunks end to end (log-mel + {args.model} encoder + prefill + "
                        f"{args.new_tokens}-token greedy decode with timestamp-pair rules"
                        + (" + DTW word timing of every window at token level" if getattr(args, "align", False) else "")
                        + "), random-init weights",
            "chunks_per_gpu_per_step": args.clips, "new_tokens": args.new_tokens, "prompt_len": len(PROMPT),
            "parallelism": f"dp{args.gpus} (independent chunks, no collective on the path)",
            "l2": "working set per decode step (cross K/V of all slots) is far larger than the 126 MB L2"}


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="large-v3")
    ap.add_argument("--clips", type=int, default=384,
                    help="30 s chunks per GPU per step = decode rows per step (384 slots hold 122 GB of KV cache)")
    ap.add_argument("--max-clips", type=int, default=32, help="windows per encoder call (32: fuller tile waves than 16)")
    ap.add_argument("--new-tokens", type=int, default=224)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cfg4", action="store_true", help="skip the 1 h strong-scaling extra (cfg4_strong_rtfx)")
    ap.add_argument("--steps-per-poll", type=int, default=8)
    ap.add_argument("--align", action="store_true",
                    help="also run the DTW word-timing alignment on every finished window (token-level words); "
                         "not part of the headline workload, named in config.workload when on")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch.distributed as dist
    from whisperdrz_b200 import synth
    from whisperdrz_b200.alignment import token_aligner
    from whisperdrz_b200.dims import ModelDimensions
    from whisperdrz_b200.engine import Engine
    from whisperdrz_b200.rules import timestamp_tables
    from whisperdrz_b200.transcriber import Transcriber
    from whisperdrz_b200.weights import init_state_dict

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    dims = ModelDimensions.from_name(args.model)
    sd = init_state_dict(dims, 0)
    eng = Engine(dims, sd, dtype=torch.bfloat16, device=dev, n_slots=args.clips, max_clips=min(args.max_clips, args.clips),
                 max_rows=max(args.clips, 128, 4096 if args.align else 0),
                 tables=timestamp_tables(dims.n_vocab))
    audio_host = torch.from_numpy(synth.clips([1000 * rank + i + 1 for i in range(args.clips)])).pin_memory()
    audio_dev = audio_host.to(dev)

    def one_step(src):
        tr = Transcriber(eng, max_new_tokens=args.new_tokens, max_continuations=0,
                         device_rules=True, steps_per_poll=args.steps_per_poll,
                         aligner=token_aligner if args.align else None)
        for i in range(args.clips):
            tr.pending_chunks.append({"audio": src[i], "id": f"chunk_{i}", "duration": 30.0, "offset": 0.0})
        out = []
        while tr.pending_chunks or any(s.status != "ready" for s in tr.states):
            r = tr._run_batched_inference()
            if r:
                out.extend(r)
        return tr, out

    def timed(src, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = eng.launch_count()
        a.record()
        n_tok = 0
        dsteps = 0
        for _ in range(steps):
            tr, out = one_step(src)
            n_tok += sum(len(r["tokens"]) for r in out)
            dsteps += tr.steps
        b.record()
        torch.cuda.synchronize()
        eng.device_status()        # raises if any kernel of the timed steps reported an error: no number then
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.barrier()
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), n_tok, dsteps, eng.launch_count() - l0

    for _ in range(args.warmup):
        one_step(audio_dev)
    sampler = ClockSampler(local)
    sampler.start()
    ms, n_tok, dsteps, launches = timed(audio_dev, args.steps)
    clocks = sampler.summary()
    ms_e2e, n_tok_e, dsteps_e, _ = timed(audio_host, args.steps)

    audio_s = 30.0 * args.clips * args.steps * world
    value = audio_s / (ms / 1e3)
    e2e = audio_s / (ms_e2e / 1e3)
    rule_bytes = 128 * n_tok_e // max(args.steps, 1)
    h2d = args.clips * 480000 * 4 + rule_bytes + 8 * n_tok_e // max(args.steps, 1)
    d2h = 4 * n_tok_e // max(args.steps, 1)

    # roofline of the dominant kernel, from one extra profiled step (kernel by kernel outside the graph, the whole batch
    # on one stream: the timed steps overlap two half-batches, where a launch's duration is not the kernel's alone)
    eng.profile(True)
    one_step(audio_dev)
    prof = eng.profile_read()
    eng.profile(False)
    peak, peak_kind = peaks()
    ca = prof["cross_attn"]
    # dram read+write per row per launch of this kernel from an ncu capture of a 32-row launch
    # (245.972 MB read + 4.381 MB written); every row has its own K/V, so traffic grows linearly with rows
    traffic_per_row = (245.971712e6 + 4.381184e6) / 32
    per_launch_ms = ca["ms"] / max(ca["launches"], 1)
    per_launch_bytes = ca["work"] / max(ca["launches"], 1)
    achieved = per_launch_bytes / (per_launch_ms * 1e-3) / 1e9 if per_launch_ms > 0 else 0.0
    shares = {k: round(v["ms"], 3) for k, v in prof.items()}

    # BASELINE config 4 as an extra, strong-scaling key: ONE hour of long-form audio, cut by the 30 s split into 120
    # chunks that are sharded over the ranks, decoded and gathered on rank 0 for stitching
    cfg4 = None
    if not args.no_cfg4:
        from whisperdrz_b200.sharding import transcribe_sharded
        hour = torch.from_numpy(synth.long_form(3, 3600.0)).pin_memory()

        def run_hour():
            tr = Transcriber(eng, max_new_tokens=args.new_tokens, max_continuations=0, device_rules=True,
                             steps_per_poll=args.steps_per_poll)
            return transcribe_sharded(tr, hour, rank, world)
        run_hour()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = run_hour()
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        eng.device_status()
        if rank == 0:
            cfg4 = {"cfg4_strong_rtfx": 3600.0 / float(dt.item()), "cfg4_chunks_gathered": len(res.raw_chunks),
                    "cfg4_seconds": float(dt.item())}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args),
                "clocks": clocks,
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
                "gpu_launches": int(launches),
                "decode_tokens_per_s": n_tok * world / (ms / 1e3),
                "roofline": {"kernel": "attn_dec_stream_kernel (decode cross-attention)", "bound": "hbm",
                             "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                             "frac": achieved / peak,
                             "traffic": traffic_per_row * per_launch_bytes / (2.0 * 1500 * 1280 * 2),
                             "bytes_per_launch": per_launch_bytes, "ms_per_launch": per_launch_ms},
                "kernel_ms_one_step": shares}
        if cfg4:
            line.update(cfg4)
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            arm = CpuArm(sd, dims, args.new_tokens)
            arm.decode_steps(1)                         # warm-up: page in the weights, spin up the thread pool
            enc = [arm.encoder_side()]
            dec = arm.decode_steps(arm.per_step)
            full = arm.seconds_per_unit(enc, dec, arm.per_step)
            line["cpu_baseline"] = {"value": 30.0 / full, "unit": UNIT, "cores": cores, "kind": arm.kind,
                                    "sample": arm.describe(arm.per_step, 1)}
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
