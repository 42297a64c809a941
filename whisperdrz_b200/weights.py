"""Seeded random-init weights with the reference's state_dict names and shapes.

The reference leaves ``decoder.positional_embedding`` uninitialised
(``torch.empty``, src/whisperdrz/model.py:494) and relies on checkpoints that are
not available offline, so every tensor here is drawn explicitly from a
per-tensor CPU generator.  The same (dims, seed) gives bit-identical tensors
on every machine with the same torch build, which is what lets golden vectors
made with the reference on one box be compared on another.

Tensor names and shapes follow the reference modules:
encoder (model.py:437-461), decoder (model.py:478-530), attention
(model.py:258-261: key has no bias), MLP (model.py:387-393).
"""
from __future__ import annotations

import math
import zlib

import numpy as np
import torch

from .dims import ModelDimensions


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """Encoder positional table (model.py:208-214), fp32 [length, channels]."""
    inc = np.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    t = torch.arange(length)[:, None] * inv[None, :]
    return torch.cat([torch.sin(t), torch.cos(t)], dim=1)


def _draw(name: str, shape, std: float, seed: int, mean: float = 0.0) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed((zlib.crc32(name.encode()) * 1000003 + seed) % (2**63 - 1))
    t = torch.empty(shape, dtype=torch.float32)
    t.normal_(0.0, 1.0, generator=g)
    return t.mul_(std).add_(mean)


def _block(sd: dict, p: str, d: int, cross: bool, seed: int) -> None:
    names = ["attn"] + (["cross_attn"] if cross else [])
    for a in names:
        s = 1.0 / math.sqrt(d)
        sd[f"{p}.{a}.query.weight"] = _draw(f"{p}.{a}.query.weight", (d, d), s, seed)
        sd[f"{p}.{a}.query.bias"] = _draw(f"{p}.{a}.query.bias", (d,), 0.02, seed)
        sd[f"{p}.{a}.key.weight"] = _draw(f"{p}.{a}.key.weight", (d, d), s, seed)
        sd[f"{p}.{a}.value.weight"] = _draw(f"{p}.{a}.value.weight", (d, d), s, seed)
        sd[f"{p}.{a}.value.bias"] = _draw(f"{p}.{a}.value.bias", (d,), 0.02, seed)
        sd[f"{p}.{a}.out.weight"] = _draw(f"{p}.{a}.out.weight", (d, d), 0.5 * s, seed)
        sd[f"{p}.{a}.out.bias"] = _draw(f"{p}.{a}.out.bias", (d,), 0.02, seed)
        sd[f"{p}.{a}_ln.weight"] = _draw(f"{p}.{a}_ln.weight", (d,), 0.05, seed, 1.0)
        sd[f"{p}.{a}_ln.bias"] = _draw(f"{p}.{a}_ln.bias", (d,), 0.05, seed)
    sd[f"{p}.mlp.0.weight"] = _draw(f"{p}.mlp.0.weight", (4 * d, d), 1.0 / math.sqrt(d), seed)
    sd[f"{p}.mlp.0.bias"] = _draw(f"{p}.mlp.0.bias", (4 * d,), 0.02, seed)
    sd[f"{p}.mlp.2.weight"] = _draw(f"{p}.mlp.2.weight", (d, 4 * d), 0.5 / math.sqrt(4 * d), seed)
    sd[f"{p}.mlp.2.bias"] = _draw(f"{p}.mlp.2.bias", (d,), 0.02, seed)
    sd[f"{p}.mlp_ln.weight"] = _draw(f"{p}.mlp_ln.weight", (d,), 0.05, seed, 1.0)
    sd[f"{p}.mlp_ln.bias"] = _draw(f"{p}.mlp_ln.bias", (d,), 0.05, seed)


def init_state_dict(dims: ModelDimensions, seed: int = 0) -> dict[str, torch.Tensor]:
    """fp32 CPU state_dict loadable into the reference ``WhisperDRZ`` with
    ``load_state_dict(strict=True)``."""
    sd: dict[str, torch.Tensor] = {}
    da, dt = dims.n_audio_state, dims.n_text_state
    sd["encoder.conv1.weight"] = _draw("encoder.conv1.weight", (da, dims.n_mels, 3),
                                       1.0 / math.sqrt(3 * dims.n_mels), seed)
    sd["encoder.conv1.bias"] = _draw("encoder.conv1.bias", (da,), 0.02, seed)
    sd["encoder.conv2.weight"] = _draw("encoder.conv2.weight", (da, da, 3),
                                       1.0 / math.sqrt(3 * da), seed)
    sd["encoder.conv2.bias"] = _draw("encoder.conv2.bias", (da,), 0.02, seed)
    sd["encoder.positional_embedding"] = sinusoids(dims.n_audio_ctx, da)
    for i in range(dims.n_audio_layer):
        _block(sd, f"encoder.blocks.{i}", da, False, seed)
    sd["encoder.ln_post.weight"] = _draw("encoder.ln_post.weight", (da,), 0.05, seed, 1.0)
    sd["encoder.ln_post.bias"] = _draw("encoder.ln_post.bias", (da,), 0.05, seed)

    sd["decoder.token_embedding.weight"] = _draw("decoder.token_embedding.weight",
                                                 (dims.n_vocab, dt), 0.02, seed)
    sd["decoder.positional_embedding"] = _draw("decoder.positional_embedding",
                                               (dims.n_text_ctx, dt), 0.02, seed)
    for i in range(dims.n_text_layer):
        _block(sd, f"decoder.blocks.{i}", dt, True, seed)
    sd["decoder.ln.weight"] = _draw("decoder.ln.weight", (dt,), 0.05, seed, 1.0)
    sd["decoder.ln.bias"] = _draw("decoder.ln.bias", (dt,), 0.05, seed)
    return sd


def n_params(sd: dict[str, torch.Tensor]) -> int:
    return sum(v.numel() for k, v in sd.items() if k != "encoder.positional_embedding")
