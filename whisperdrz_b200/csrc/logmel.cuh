// Fused log-mel front end: framing with reflect padding, periodic Hann window,
// 400-point real DFT (201 bins) by direct summation against a 400-entry
// twiddle table, power, slaney mel filterbank, log10 - all in one kernel per
// 32-frame tile - followed by a finalize pass that applies the per-clip
// (max - 8) floor, the (x + 4) / 4 scaling, the window offset and the -1.5
// padding.  Follows LogMelSpectrogram (src/whisperdrz/audio.py:108-156) and the
// window slicing of Transcriber._prefill_slots (transcriber.py:1062-1072).
//
// HBM-bound stage: 1.92 MB of audio read and 1.536 MB of mel written per 30 s
// clip; the ~1 GFLOP of DFT arithmetic per clip runs on the CUDA cores.
#pragma once
#include "common.cuh"

namespace wdz {

constexpr int MEL_NFFT = 400;
constexpr int MEL_HOP = 160;
constexpr int MEL_BINS = 201;
constexpr int MEL_FT = 32;        // frames per CTA
constexpr int MEL_MAX_FRAMES = 3000;
constexpr int MEL_SPAN = (MEL_FT - 1) * MEL_HOP + MEL_NFFT;  // samples a tile touches
constexpr int MEL_PS_LD = 205;    // leading dimension of the power tile (odd: no bank conflicts)

struct MelTables {
  const float2* twiddle;  // [400] (cos, sin)(2 pi j / 400)
  const float* window;    // [400] periodic Hann
  const float* fb;        // [201, n_mels] filterbank
  const int* band_lo;     // [n_mels] first bin with non-zero weight
  const int* band_hi;     // [n_mels] one past the last
};

__device__ __forceinline__ int float_to_ordered(float f) {
  int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) {
  return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

// raw [B, n_mels, 3000] = log10(max(mel, 1e-10)); clipmax[b] = ordered-int max over valid frames.
__global__ void __launch_bounds__(256)
logmel_raw_kernel(const float* __restrict__ audio, int64_t audio_stride,
                  const int* __restrict__ n_samples, MelTables tb, int n_mels,
                  float* __restrict__ raw, int* __restrict__ clipmax) {
  extern __shared__ float smem[];
  float* xs = smem;                                   // [MEL_SPAN]
  float* ps = xs + MEL_SPAN;                          // [MEL_FT][MEL_PS_LD]
  float2* tw = reinterpret_cast<float2*>(ps + MEL_FT * MEL_PS_LD);  // [400], pre-multiplied by nothing
  float* win = reinterpret_cast<float*>(tw + MEL_NFFT);            // [400]
  __shared__ float red[8];

  const int b = blockIdx.y;
  const int f0 = blockIdx.x * MEL_FT;
  const int N = n_samples[b];
  const int n_frames = min(N / MEL_HOP, MEL_MAX_FRAMES);
  if (f0 >= n_frames) return;
  const float* a = audio + (int64_t)b * audio_stride;
  const int tid = threadIdx.x;

  for (int i = tid; i < MEL_SPAN; i += 256) {
    int s = f0 * MEL_HOP - MEL_NFFT / 2 + i;
    if (s < 0) s = -s;
    if (s >= N) s = 2 * (N - 1) - s;
    xs[i] = (s >= 0 && s < N) ? a[s] : 0.0f;
  }
  for (int i = tid; i < MEL_NFFT; i += 256) {
    tw[i] = tb.twiddle[i];
    win[i] = tb.window[i];
  }
  __syncthreads();

  // DFT: thread k < 201 owns bin k, eight frames at a time.
  if (tid < MEL_BINS) {
    const int k = tid;
    for (int fg = 0; fg < MEL_FT; fg += 8) {
      float re[8], im[8];
#pragma unroll
      for (int f = 0; f < 8; ++f) re[f] = im[f] = 0.0f;
      int idx = 0;
      const float* xb = xs + fg * MEL_HOP;
      for (int n = 0; n < MEL_NFFT; ++n) {
        const float2 t = tw[idx];
        const float w = win[n];
        const float c = t.x * w, s = t.y * w;
#pragma unroll
        for (int f = 0; f < 8; ++f) {
          const float x = xb[f * MEL_HOP + n];
          re[f] = fmaf(x, c, re[f]);
          im[f] = fmaf(x, s, im[f]);
        }
        idx += k;
        if (idx >= MEL_NFFT) idx -= MEL_NFFT;
      }
#pragma unroll
      for (int f = 0; f < 8; ++f) ps[(fg + f) * MEL_PS_LD + k] = re[f] * re[f] + im[f] * im[f];
    }
  }
  __syncthreads();

  // mel + log10 into a [n_mels][MEL_FT + 1] tile that reuses the sample buffer.
  float* os = xs;
  float local_max = -INFINITY;
  for (int i = tid; i < n_mels * MEL_FT; i += 256) {
    const int m = i % n_mels, f = i / n_mels;
    const int lo = tb.band_lo[m], hi = tb.band_hi[m];
    float acc = 0.0f;
    for (int k = lo; k < hi; ++k) acc = fmaf(ps[f * MEL_PS_LD + k], tb.fb[k * n_mels + m], acc);
    const float L = log10f(fmaxf(acc, 1e-10f));
    os[m * (MEL_FT + 1) + f] = L;
    if (f0 + f < n_frames) local_max = fmaxf(local_max, L);
  }
  __syncthreads();
  for (int i = tid; i < n_mels * MEL_FT; i += 256) {
    const int m = i / MEL_FT, f = i % MEL_FT;
    if (f0 + f < n_frames)
      raw[((int64_t)b * n_mels + m) * MEL_MAX_FRAMES + f0 + f] = os[m * (MEL_FT + 1) + f];
  }
  local_max = warp_max(local_max);
  if ((tid & 31) == 0) red[tid >> 5] = local_max;
  __syncthreads();
  if (tid == 0) {
    float m = red[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    if (m > -INFINITY) atomicMax(clipmax + b, float_to_ordered(m));
  }
}

__global__ void logmel_init_max_kernel(int* clipmax, int B) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B) clipmax[i] = INT_MIN;
}

// out [B, n_mels, 3000]: window starting at frame_offset[b]; -1.5 past the clip.
__global__ void __launch_bounds__(256)
logmel_finalize_kernel(const float* __restrict__ raw, const int* __restrict__ clipmax,
                       const int* __restrict__ n_samples, const int* __restrict__ frame_offset,
                       int n_mels, float* __restrict__ out) {
  const int b = blockIdx.z, m = blockIdx.y;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= MEL_MAX_FRAMES) return;
  const int n_frames = min(n_samples[b] / MEL_HOP, MEL_MAX_FRAMES);
  const int f = j + (frame_offset ? frame_offset[b] : 0);
  float v = -1.5f;
  if (f >= 0 && f < n_frames) {
    const float floor_v = ordered_to_float(clipmax[b]) - 8.0f;
    const float L = raw[((int64_t)b * n_mels + m) * MEL_MAX_FRAMES + f];
    v = (fmaxf(L, floor_v) + 4.0f) / 4.0f;
  }
  out[((int64_t)b * n_mels + m) * MEL_MAX_FRAMES + j] = v;
}

inline size_t logmel_smem_bytes() {
  return sizeof(float) * (MEL_SPAN + MEL_FT * MEL_PS_LD + 2 * MEL_NFFT + MEL_NFFT);
}

}  // namespace wdz
