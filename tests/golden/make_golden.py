"""Generate the golden vectors under tests/golden/ by running the reference.

Run where the reference is mounted:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py [--large]

It imports the reference's own ``LogMelSpectrogram`` and ``WhisperDRZ``
(unmodified), loads the seeded weights of ``whisperdrz_b200.weights`` into
them and records small slices of what they compute on the seeded synthetic
clips of ``whisperdrz_b200.synth``.  Only slices are stored (a few hundred KB);
the slicing pattern is stored with them.  ``--large`` adds the full-size
large-v3 case (224 greedy tokens from a 4-token prompt with EOS suppressed);
it needs about 14 GB of RAM and a few minutes of CPU.
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


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--large", action="store_true")
    ap.add_argument("--skip-small", action="store_true")
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
    print("done")
