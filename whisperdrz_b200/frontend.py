"""Constant tables of the log-mel kernel, computed once on the host in float64:
the 400-point twiddle table, the periodic Hann window and the slaney mel
filterbank (the quantities ``LogMelSpectrogram`` holds as ``window`` and
``mel_scale.fb``, src/whisperdrz/audio.py:98-106)."""
from __future__ import annotations

import math

import numpy as np

N_FFT = 400
N_BINS = N_FFT // 2 + 1


def twiddle() -> np.ndarray:
    j = np.arange(N_FFT, dtype=np.float64)
    ang = 2.0 * np.pi * j / N_FFT
    return np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


def hann_periodic() -> np.ndarray:
    n = np.arange(N_FFT, dtype=np.float64)
    return (0.5 - 0.5 * np.cos(2.0 * np.pi * n / N_FFT)).astype(np.float32)


def _hz_to_mel(f):
    f = np.asarray(f, dtype=np.float64)
    lin = f / (200.0 / 3)
    logstep = math.log(6.4) / 27.0
    log_part = 15.0 + np.log(np.maximum(f, 1e-30) / 1000.0) / logstep
    return np.where(f >= 1000.0, log_part, lin)


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    logstep = math.log(6.4) / 27.0
    return np.where(m >= 15.0, 1000.0 * np.exp(logstep * (m - 15.0)), m * (200.0 / 3))


def mel_filterbank(n_mels: int = 128, sample_rate: int = 16000):
    """Returns (fb f32 [201, n_mels], band_lo int32 [n_mels], band_hi int32 [n_mels]):
    slaney-scale triangles with slaney (area) normalisation, and per filter the
    half-open range of DFT bins with non-zero weight."""
    freqs = np.linspace(0.0, sample_rate / 2.0, N_BINS)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(sample_rate / 2.0), n_mels + 2))
    diff = pts[1:] - pts[:-1]
    slopes = pts[None, :] - freqs[:, None]
    down = -slopes[:, :-2] / diff[:-1]
    up = slopes[:, 2:] / diff[1:]
    fb = np.maximum(0.0, np.minimum(down, up))
    fb *= (2.0 / (pts[2:] - pts[:-2]))[None, :]
    fb = fb.astype(np.float32)
    lo = np.zeros(n_mels, np.int32)
    hi = np.zeros(n_mels, np.int32)
    for m in range(n_mels):
        nz = np.nonzero(fb[:, m])[0]
        if len(nz):
            lo[m], hi[m] = nz[0], nz[-1] + 1
    return fb, lo, hi
