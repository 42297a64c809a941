"""Seeded synthetic audio standing in for real recordings.

No dataset or checkpoint is reachable offline, so every test and benchmark
input is generated here from a seed: 16 kHz mono float32 clips of Gaussian
noise plus a few sinusoids, long-form audio built from such segments separated
by near-silence, and request-duration / arrival draws for the serving case.
"""
from __future__ import annotations

import numpy as np

from .dims import SAMPLE_RATE


def clip(seed: int, seconds: float = 30.0, noise_sigma: float = 0.05,
         n_tones: int = 3, tone_amp: float = 0.1) -> np.ndarray:
    """One clip: N(0, sigma^2) noise + ``n_tones`` sinusoids in 200-3000 Hz."""
    rng = np.random.default_rng(seed)
    n = int(round(seconds * SAMPLE_RATE))
    x = rng.normal(0.0, noise_sigma, n)
    t = np.arange(n, dtype=np.float64) / SAMPLE_RATE
    for _ in range(n_tones):
        f = rng.uniform(200.0, 3000.0)
        ph = rng.uniform(0.0, 2 * np.pi)
        x += tone_amp * np.sin(2 * np.pi * f * t + ph)
    return x.astype(np.float32)


def clips(seeds, seconds: float = 30.0) -> np.ndarray:
    return np.stack([clip(s, seconds) for s in seeds])


def long_form(seed: int, total_seconds: float) -> np.ndarray:
    """Concatenated 2-20 s noise+tone segments separated by 0.2-2 s of
    sigma=0.001 noise, trimmed to ``total_seconds``."""
    rng = np.random.default_rng(seed)
    out, have, k = [], 0, 0
    want = int(round(total_seconds * SAMPLE_RATE))
    while have < want:
        seg = clip(int(rng.integers(1 << 30)) + k, float(rng.uniform(2.0, 20.0)))
        gap = rng.normal(0.0, 0.001, int(rng.uniform(0.2, 2.0) * SAMPLE_RATE)).astype(np.float32)
        out += [seg, gap]
        have += len(seg) + len(gap)
        k += 1
    return np.concatenate(out)[:want]


def request_durations(seed: int, n: int, lo: float = 5.0, hi: float = 600.0) -> np.ndarray:
    """Log-uniform request durations in seconds."""
    rng = np.random.default_rng(seed)
    return np.exp(rng.uniform(np.log(lo), np.log(hi), n))


def poisson_arrivals(seed: int, n: int, rate_per_s: float) -> np.ndarray:
    """Arrival times (s) of a Poisson process of the given rate."""
    rng = np.random.default_rng(seed)
    return np.cumsum(rng.exponential(1.0 / rate_per_s, n))


def decode_lengths(seed: int, n: int, max_total: int = 448):
    """Prompt lengths U{4..64}, generated lengths U{32..448}, clipped so that
    prompt + generated <= max_total; prompt ids U{0..49999}."""
    rng = np.random.default_rng(seed)
    p = rng.integers(4, 65, n)
    g = np.minimum(rng.integers(32, 449, n), max_total - p)
    prompts = [rng.integers(0, 50000, int(pi)).astype(np.int64) for pi in p]
    return p.astype(np.int64), g.astype(np.int64), prompts
