"""Generate the golden vectors under tests/golden/ by running the reference.

Run where the reference is mounted:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py [--large]

It imports the reference's own ``LogMelSpectrogram`` and ``WhisperDRZ``
(unmodified), loads the seeded weights of ``whisperdrz_b200.weights`` into
them and records small slices of what they compute on the seeded synthetic
clips of ``whisperdrz_b200.synth``.  Only slices are stored (a few hundred KB);
the slicing pattern is stored with them.  ``--large`` adds the full-size
large-v3 case (224 greedy tokens from a 4-token prompt with EOS suppressed);
it needs about 14 GB of RAM and a few minutes of CPU.  ``--large-rows`` records
the full-size ragged multi-row decode case (32 slots, prompts of 4..420 tokens,
24 teacher-forced steps; see ``rows_golden``); about 25 GB of RAM.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from whisperdrz_b200 import synth  # noqa: E402
from whisperdrz_b200.dims import ModelDimensions, TOK_EOT  # noqa: E402
from whisperdrz_b200.weights import init_state_dict  # noqa: E402

from whisperdrz.audio import LogMelSpectrogram  # noqa: E402  (the reference)
from whisperdrz.config import Config, ModelDimensions as RefDims  # noqa: E402
from whisperdrz.model import WhisperDRZ  # noqa: E402

PROMPT = [50258, 50259, 50360, 50365]


def ref_model(dims: ModelDimensions, seed: int):
    m = WhisperDRZ(RefDims(**dims.as_dict()), config=Config()).float().eval()
    sd = init_state_dict(dims, seed)
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("speaker" in k or "timing" in k for k in missing), missing
    return m


def mel_golden():
    tomel = LogMelSpectrogram(128)
    out = {}
    for name, seed, secs in [("clip30", 1, 30.0), ("clip7", 5, 7.3), ("clip1", 9, 1.0)]:
        a = torch.from_numpy(synth.clip(seed, secs))
        mel = tomel(a.unsqueeze(0), target_frames=3000)[0]  # [128, 3000], -1.5 padded
        out[f"{name}_seed"] = np.int64(seed)
        out[f"{name}_secs"] = np.float64(secs)
        out[f"{name}_cols"] = np.arange(0, 3000, 37)
        out[f"{name}_mel"] = mel[:, ::37].numpy()
        out[f"{name}_sum"] = np.float64(mel.double().sum().item())
    return out


@torch.inference_mode()
def model_golden(name: str, n_steps: int, seed: int = 0, clip_seeds=(1,), logit_stride: int = 97,
                 keep_steps=None):
    dims = ModelDimensions.from_name(name)
    m = ref_model(dims, seed)
    tomel = LogMelSpectrogram(dims.n_mels)
    audio = torch.from_numpy(synth.clips(clip_seeds))
    mel = tomel(audio, target_frames=3000)
    t0 = time.time()
    xa = m.encoder(mel)
    B = xa.shape[0]
    n_slots = B + 2
    slots = torch.arange(1, B + 1)  # deliberately not slot 0
    m.decoder.cache_embedding_weight(torch.float32)
    self_kv, cross_kv = m.create_flash_kv(n_slots, max_tokens=dims.n_text_ctx)
    prompt = torch.tensor([[min(t, dims.n_vocab - 1) for t in PROMPT]] * B)
    logits = m.prefill_flash(prompt, xa, self_kv, cross_kv, slots)[:, -1]
    eot = min(TOK_EOT, dims.n_vocab - 1)
    toks, kept = [], {}
    keep_steps = set(range(n_steps)) if keep_steps is None else set(keep_steps)
    for step in range(n_steps):
        if step in keep_steps:
            kept[step] = logits[:, ::logit_stride].clone()
        lg = logits.clone()
        lg[:, eot] = float("-inf")
        nxt = lg.argmax(-1)
        toks.append(nxt.clone())
        pos = self_kv[0].seq_lens[slots]
        logits = m.decoder.forward_flash(nxt[:, None], self_kv, cross_kv, pos, slot_indices=slots)[:, 0]
    print(f"{name}: encoder+decode {time.time() - t0:.1f}s")
    out = {
        "seed": np.int64(seed),
        "clip_seeds": np.asarray(clip_seeds),
        "prompt": prompt.numpy(),
        "xa_rows": np.arange(0, 1500, 50),
        "xa": xa[:, ::50].numpy(),
        "xa_sqsum": np.float64((xa.double() ** 2).sum().item()),
        "tokens": torch.stack(toks, 1).numpy(),
        "logit_stride": np.int64(logit_stride),
        "logit_steps": np.asarray(sorted(kept)),
        "logits": torch.stack([kept[s] for s in sorted(kept)], 1).numpy(),
        "final_seq_lens": self_kv[0].seq_lens.numpy(),
    }
    return out


ROWS_N, ROWS_STEPS, ROWS_GROUP, ROWS_STRIDE = 32, 24, 8, 97


def rows_inputs(n_rows: int = ROWS_N, seed: int = 2):
    """Seeded inputs of the ragged multi-row case, shared with the GPU test:
    encoder states xa_i ~ N(0, 1) [1500, d] (seed 100 + i), prompt lengths
    U{4..64} with ids U{0..49999} (``synth.decode_lengths``), except that the last
    four rows carry 150/250/350/420-token prompts so that deep caches are covered."""
    p, _, prompts = synth.decode_lengths(seed, n_rows)
    rng = np.random.default_rng(seed + 1)
    for j, n in enumerate((150, 250, 350, 420)):
        prompts[n_rows - 4 + j] = rng.integers(0, 50000, n).astype(np.int64)
    return prompts


def rows_xa(i: int, d: int) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(100 + i)
    return torch.empty(1500, d, dtype=torch.float32).normal_(0.0, 1.0, generator=g)


@torch.inference_mode()
def rows_golden(name: str = "large-v3", seed: int = 0):
    """The batched ragged decode of the throughput benchmark at full size, from
    the unmodified reference on CPU in fp32: every row is prefilled on its own
    (the reference's ``prefill_flash`` takes rectangular prompts), then
    ``ROWS_STEPS`` decode steps run ``ROWS_GROUP`` rows at a time through
    ``decoder.forward_flash`` at each row's own depth.  The token fed at every step
    is the reference's greedy choice (EOS suppressed) and is stored, so that the
    engine can be teacher-forced with it.  Stored per (row, step): every
    ``ROWS_STRIDE``-th logit, the full-row RMS and the arg-max id."""
    dims = ModelDimensions.from_name(name)
    m = ref_model(dims, seed)
    m.decoder.cache_embedding_weight(torch.float32)
    prompts = rows_inputs()
    eot = min(TOK_EOT, dims.n_vocab - 1)
    n_keep = len(range(0, dims.n_vocab, ROWS_STRIDE))
    logits_k = np.zeros((ROWS_N, ROWS_STEPS + 1, n_keep), np.float32)
    rms = np.zeros((ROWS_N, ROWS_STEPS + 1), np.float64)
    fed = np.zeros((ROWS_N, ROWS_STEPS + 1), np.int64)
    t0 = time.time()
    for g0 in range(0, ROWS_N, ROWS_GROUP):
        rows = list(range(g0, g0 + ROWS_GROUP))
        self_kv, cross_kv = m.create_flash_kv(ROWS_GROUP, max_tokens=dims.n_text_ctx)
        cur = []
        for j, r in enumerate(rows):
            xa = rows_xa(r, dims.n_audio_state)[None]
            pr = torch.from_numpy(prompts[r])[None]
            lg = m.prefill_flash(pr, xa, self_kv, cross_kv, torch.tensor([j]))[0, -1]
            cur.append(lg)
        logits = torch.stack(cur)
        slots = torch.arange(ROWS_GROUP)
        for step in range(ROWS_STEPS + 1):
            logits_k[rows, step] = logits[:, ::ROWS_STRIDE].numpy()
            rms[rows, step] = logits.double().pow(2).mean(-1).sqrt().numpy()
            lg = logits.clone()
            lg[:, eot] = float("-inf")
            nxt = lg.argmax(-1)
            fed[rows, step] = nxt.numpy()
            if step == ROWS_STEPS:
                break
            pos = self_kv[0].seq_lens[slots]
            logits = m.decoder.forward_flash(nxt[:, None], self_kv, cross_kv, pos, slot_indices=slots)[:, 0]
        print(f"rows {g0}..{g0 + ROWS_GROUP - 1}: {time.time() - t0:.1f}s", flush=True)
        del self_kv, cross_kv
    return {"seed": np.int64(seed), "stride": np.int64(ROWS_STRIDE), "logits": logits_k, "rms": rms,
            "tokens": fed, "prompt_lens": np.asarray([len(p) for p in prompts])}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--large", action="store_true")
    ap.add_argument("--skip-small", action="store_true")
    ap.add_argument("--large-rows", action="store_true")
    args = ap.parse_args()
    torch.manual_seed(0)
    if not args.skip_small:
        np.savez_compressed(os.path.join(HERE, "mel.npz"), **mel_golden())
        np.savez_compressed(os.path.join(HERE, "model_test_small.npz"),
                            **model_golden("test-small", 12, clip_seeds=(1, 2)))
        np.savez_compressed(os.path.join(HERE, "model_test_tiny.npz"),
                            **model_golden("test-tiny", 12, clip_seeds=(3,), logit_stride=7))
    if args.large:
        np.savez_compressed(os.path.join(HERE, "model_large_v3_cfg1.npz"),
                            **model_golden("large-v3", 224, clip_seeds=(1,), logit_stride=997,
                                           keep_steps=(0, 1, 2, 50, 100, 150, 223)))
    if args.large_rows:
        np.savez_compressed(os.path.join(HERE, "model_large_v3_rows.npz"), **rows_golden())
    print("done")
