"""Data-parallel sharding of independent chunks over GPUs (one process per GPU).

The reference is single-process (no torch.distributed anywhere).  A 30 s chunk
(src/whisperdrz/transcriber.py:784-793) is an independent unit, so N engines run
shared-nothing on replicated weights: rank r takes chunks r, r + N, ...; no
collective touches the data path; finished result dicts are gathered to rank 0
on the host and stitched in chunk order (transcriber.py:803-810)."""
from __future__ import annotations

import numpy as np
import torch

from .dims import SAMPLE_RATE


def split_chunks(audio, max_audio_length: float = 30.0) -> list[dict]:
    """The reference's fixed 30 s split (transcriber.py:780-793)."""
    if isinstance(audio, np.ndarray):
        audio = torch.from_numpy(audio)
    audio = audio.squeeze()
    n = int(max_audio_length * SAMPLE_RATE)
    out = []
    for i, start in enumerate(range(0, len(audio), n)):
        end = min(start + n, len(audio))
        out.append({"audio": audio[start:end], "id": f"chunk_{i}", "duration": (end - start) / SAMPLE_RATE,
                    "offset": start / SAMPLE_RATE})
    return out


def shard(chunks: list, rank: int, world: int) -> list:
    return chunks[rank::world]


def gather_results(local: list[dict], rank: int, world: int) -> list[dict] | None:
    """Host-side gather of result dicts to rank 0 (None elsewhere), ordered by chunk id."""
    if world == 1:
        merged = list(local)
    else:
        import torch.distributed as dist
        bucket = [None] * world if rank == 0 else None
        dist.gather_object(local, bucket, dst=0)
        if rank != 0:
            return None
        merged = [r for part in bucket for r in part]
    merged.sort(key=lambda r: int(str(r.get("id", "chunk_0")).split("_")[-1]))
    return merged


def transcribe_sharded(transcriber, audio, rank: int, world: int):
    """Every rank calls this with the same audio; rank 0 gets the stitched
    ``TranscribeResults``, the others None."""
    mine = shard(split_chunks(audio, transcriber.max_audio_length), rank, world)
    transcriber.pending_chunks.extend(mine)
    local = list(transcriber.flush())
    merged = gather_results(local, rank, world)
    return None if merged is None else transcriber.stitch(merged)
