"""B200-native transcription hot path of whisperdrz: fused log-mel front end,
Whisper-large-v3 encoder and batched KV-cached decoder with fused logit rules,
as hand-written sm_100a CUDA behind a C ABI (include/wdz.h), driven by a
continuous-batching scheduler.

    import whisperdrz_b200
    t = whisperdrz_b200.load_model("large-v3")      # seeded random-init weights
    out = t.transcribe(audio_16khz)                 # TranscribeResults

``load_model`` has the shape of the reference's ``whisperdrz.load_model``
(src/whisperdrz/__init__.py:9-22): a model name or checkpoint path, ``lang`` and
keyword arguments of the Transcriber.
"""
from __future__ import annotations

from .dims import ModelDimensions

__all__ = ["load_model", "ModelDimensions"]


def load_model(name_or_path="large-v3", lang: str | None = "en", dtype=None, device="cuda:0",
               seed: int = 0, n_slots: int = 32, max_clips: int = 16, **kwargs):
    """Returns a ready ``Transcriber``.

    name_or_path: a shape name known to ``ModelDimensions.from_name`` (weights
    are then drawn from ``seed``; released checkpoints are not reachable
    offline), or a path to a ``.pt`` / ``.safetensors`` state_dict with the
    reference's tensor names (large-v3 shapes).  ``dtw_align=True`` (the
    reference's default, transcriber.py:525) adds word timing of every finished
    window at token level (``alignment.token_aligner``; pass ``aligner=`` for a
    tokenizer-aware one): results then carry ``word_times``."""
    import os

    import torch

    from .engine import Engine
    from .rules import timestamp_tables
    from .transcriber import Transcriber
    from .weights import init_state_dict

    dtype = dtype or torch.bfloat16
    if isinstance(name_or_path, str) and os.path.exists(name_or_path):
        if name_or_path.endswith(".safetensors"):
            from safetensors.torch import load_file
            sd = load_file(name_or_path, device="cpu")
        else:
            sd = torch.load(name_or_path, map_location="cpu", weights_only=False)
            sd = sd.get("model", sd)
        dims = ModelDimensions.from_name("large-v3")
        dims.n_text_ctx = sd["decoder.positional_embedding"].shape[0]
        dims.n_vocab = sd["decoder.token_embedding.weight"].shape[0]
    else:
        dims = ModelDimensions.from_name(name_or_path)
        sd = init_state_dict(dims, seed)
    if kwargs.pop("dtw_align", False) and "aligner" not in kwargs:
        from .alignment import token_aligner
        kwargs["aligner"] = token_aligner
    # with alignment on, room for whole chunks in one forward call (the pass then runs on the tensor cores)
    max_rows = max(n_slots, 64, 4096 if kwargs.get("aligner") is not None else 0)
    engine = Engine(dims, sd, dtype=dtype, device=device, n_slots=n_slots, max_clips=max_clips, max_rows=max_rows,
                    tables=timestamp_tables(dims.n_vocab))
    return Transcriber(engine, lang=lang, **kwargs)
