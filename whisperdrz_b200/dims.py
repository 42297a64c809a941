"""Model dimensions for the transcription hot path.

Mirrors the reference's ``ModelDimensions`` (src/whisperdrz/config.py:4-41): same
field names, same ``from_name("large-v3")`` values.  Two reduced shapes are
added for tests; they keep head_dim = 64 (the only head size the CUDA
attention kernels are written for) and the full 51866-token vocabulary layout
is optional.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict

# Audio constants (src/whisperdrz/audio.py:15-24).
SAMPLE_RATE = 16000
N_FFT = 400
HOP_LENGTH = 160
CHUNK_LENGTH = 30
N_SAMPLES = CHUNK_LENGTH * SAMPLE_RATE  # 480000
N_FRAMES = N_SAMPLES // HOP_LENGTH  # 3000

# Tokenizer constants of the multilingual large-v3 vocabulary
# (src/whisperdrz/tokenizer.py:279-295; values verified by importing it).
TOK_EOT = 50257
TOK_SOT = 50258
TOK_LANG_EN = 50259
TOK_TRANSLATE = 50359
TOK_TRANSCRIBE = 50360
TOK_NO_TIMESTAMPS = 50364
TOK_TS_BEGIN = 50365  # <|0.00|>
TOK_TS_END = 51865  # <|30.00|>, inclusive
N_VOCAB_LARGE_V3 = 51866


@dataclass
class ModelDimensions:
    n_mels: int
    n_audio_ctx: int
    n_audio_state: int
    n_audio_head: int
    n_audio_layer: int
    n_vocab: int
    n_text_ctx: int
    n_text_state: int
    n_text_head: int
    n_text_layer: int

    @classmethod
    def from_name(cls, name: str) -> "ModelDimensions":
        base = name.replace(".en", "")
        table = {
            "large-v3": cls(128, 1500, 1280, 20, 32, 51866, 448, 1280, 20, 32),
            # Reduced shapes for tests: same audio geometry (3000 mel frames ->
            # 1500 positions), fewer/narrower layers.
            "test-small": cls(128, 1500, 256, 4, 2, 51866, 448, 256, 4, 2),
            "test-tiny": cls(128, 1500, 128, 2, 2, 2048, 64, 128, 2, 2),
        }
        if base not in table:
            raise ValueError(f"Unknown model name: {name}. Supported: {list(table)}")
        return table[base]

    def as_dict(self) -> dict:
        return asdict(self)
