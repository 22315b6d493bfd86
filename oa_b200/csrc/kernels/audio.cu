// Audio DSP kernels: windowed framing for the GEMM-based STFT, spectrum magnitude, fade, mix, windowed-sinc resampling and
// the min / max waveform envelope.  Contract: Source/Private/Oa/Audio/Shader/Compute/{Transform,Signal}/*.slang of the
// reference.  The reference runs a radix-2 FFT per frame in shared memory; here the transform is a GEMM of the windowed
// frames with a [2*bins, fft] cosine / -sine basis (tensor-core shaped, any fft size), so this file only frames,
// windows and takes magnitudes.
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr float kPi = 3.14159265358979323846f;

__device__ __forceinline__ float window_value(int k, int n, int kind) {
  if (k >= n) return 0.f;
  if (kind == 3) return 1.f;
  const float phase = 2.f * kPi * (float)k / (float)n;
  if (kind == 1) return 0.54f - 0.46f * cosf(phase);
  if (kind == 2) return 0.42f - 0.5f * cosf(phase) + 0.08f * cosf(2.f * phase);
  return 0.5f * (1.f - cosf(phase));
}

// frames[(c*F + f), k] = x[c, f*hop + k - pad] * window(k); reads outside [0, samples) are zero
__global__ void stft_frame_kernel(const float* __restrict__ x, float* __restrict__ frames, int channels, long long samples, int n_frames,
                                  int fft, int hop, int win, int kind, int pad) {
  const long long total = (long long)channels * n_frames * fft;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % fft);
    const long long cf = i / fft;
    const int f = (int)(cf % n_frames), c = (int)(cf / n_frames);
    const long long sidx = (long long)f * hop + k - pad;
    const float v = (sidx >= 0 && sidx < samples) ? x[(long long)c * samples + sidx] : 0.f;
    frames[i] = v * window_value(k, win, kind);
  }
}

// spec[r, b] = |(re, im)| with reim[r, b] = re and reim[r, bins + b] = im
__global__ void spectrum_magnitude_kernel(const float* __restrict__ reim, float* __restrict__ spec, long long rows, int bins) {
  const long long total = rows * bins;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / bins;
    const int b = (int)(i % bins);
    const float re = reim[r * 2 * bins + b], im = reim[r * 2 * bins + bins + b];
    spec[i] = sqrtf(re * re + im * im);
  }
}

__global__ void audio_fade_kernel(const float* __restrict__ x, float* __restrict__ out, long long count, long long samples,
                                  long long fade_in, long long fade_out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long s = i % samples, rev = samples - 1 - s;
  float env = 1.f;
  if (fade_in > 0 && s < fade_in) env = (float)s / (float)fade_in;
  if (fade_out > 0 && rev < fade_out) env = fminf(env, (float)rev / (float)fade_out);
  out[i] = x[i] * env;
}

__global__ void audio_mix_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, long long count,
                                 float ga, float gb) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = a[i] * ga + b[i] * gb;
}

__device__ __forceinline__ float sincf_(float t) {
  if (fabsf(t) < 1e-7f) return 1.f;
  const float pt = kPi * t;
  return sinf(pt) / pt;
}

// Hann-windowed sinc interpolation at the exact rational source position j * in / out (rates reduced by their gcd);
// the sinc is scaled to the output Nyquist when down-sampling, and the taps are renormalised by their sum.
__global__ void audio_resample_kernel(const float* __restrict__ x, float* __restrict__ out, long long count, unsigned in_r, unsigned out_r,
                                      int half_width, long long in_samples, long long out_samples) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  const long long c = idx / out_samples, j = idx % out_samples;
  const long long q = j / out_r;
  const unsigned r = (unsigned)(j % out_r);
  const unsigned long long num = (unsigned long long)r * in_r;
  const long long n0 = q * in_r + (long long)(num / out_r);
  const float frac = (float)(num % out_r) / (float)out_r;
  const float scale = fminf(1.f, (float)out_r / (float)in_r), halfw = (float)half_width;
  float acc = 0.f, ksum = 0.f;
  for (int tap = -half_width; tap <= half_width; ++tap) {
    const float t = (float)tap - frac;
    if (fabsf(t) > halfw) continue;
    const float kern = scale * sincf_(scale * t) * 0.5f * (1.f + cosf(kPi * t / halfw));
    ksum += kern;
    const long long n = n0 + tap;
    if (n >= 0 && n < in_samples) acc += x[c * in_samples + n] * kern;
  }
  out[idx] = ksum > 1e-7f ? acc / ksum : 0.f;
}

// out[bin] = (min, max) over all channels of the bin's sample range; every sample belongs to exactly one bin
__global__ void audio_envelope_kernel(const float* __restrict__ x, float* __restrict__ out, int channels, long long samples, int bins) {
  const int bin = blockIdx.x * blockDim.x + threadIdx.x;
  if (bin >= bins) return;
  const long long width = samples / bins, rem = samples % bins;
  const long long begin = bin * width + (bin < rem ? bin : rem), end = begin + width + (bin < rem ? 1 : 0);
  float mn = begin < end ? x[begin] : 0.f, mx = mn;
  for (int c = 0; c < channels; ++c)
    for (long long s = begin; s < end; ++s) { const float v = x[(long long)c * samples + s]; mn = fminf(mn, v); mx = fmaxf(mx, v); }
  out[bin * 2] = mn; out[bin * 2 + 1] = mx;
}

inline int a_status() { return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH; }
inline int a_grid(long long n) { const long long g = (n + 255) / 256; return (int)(g > 148 * 64 ? 148 * 64 : g); }

}  // namespace oa

using namespace oa;

extern "C" {

int oa_audio_stft_frame(const void* x, void* frames, int channels, long long samples, int n_frames, int fft, int hop, int win, int kind,
                        int pad, void* stream) {
  if (channels <= 0 || samples <= 0 || n_frames <= 0 || fft <= 0 || hop <= 0 || win <= 0 || win > fft || kind < 0 || kind > 3) return OA_ERR_ARG;
  stft_frame_kernel<<<a_grid((long long)channels * n_frames * fft), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)frames, channels,
                                                                                                  samples, n_frames, fft, hop, win, kind, pad);
  return a_status();
}

int oa_audio_magnitude(const void* reim, void* spec, long long rows, int bins, void* stream) {
  if (rows <= 0 || bins <= 0) return OA_ERR_ARG;
  spectrum_magnitude_kernel<<<a_grid(rows * bins), 256, 0, (cudaStream_t)stream>>>((const float*)reim, (float*)spec, rows, bins);
  return a_status();
}

int oa_audio_fade(const void* x, void* out, long long count, long long samples, long long fade_in, long long fade_out, void* stream) {
  if (count <= 0 || samples <= 0) return OA_ERR_ARG;
  audio_fade_kernel<<<(int)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, count, samples, fade_in, fade_out);
  return a_status();
}

int oa_audio_mix(const void* a, const void* b, void* out, long long count, float ga, float gb, void* stream) {
  if (count <= 0) return OA_ERR_ARG;
  audio_mix_kernel<<<(int)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)a, (const float*)b, (float*)out, count, ga, gb);
  return a_status();
}

int oa_audio_resample(const void* x, void* out, int channels, long long in_samples, long long out_samples, unsigned in_r, unsigned out_r,
                      int half_width, void* stream) {
  if (channels <= 0 || in_samples <= 0 || out_samples <= 0 || in_r == 0 || out_r == 0 || half_width <= 0) return OA_ERR_ARG;
  const long long count = (long long)channels * out_samples;
  audio_resample_kernel<<<(int)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, count, in_r, out_r,
                                                                                    half_width, in_samples, out_samples);
  return a_status();
}

int oa_audio_envelope(const void* x, void* out, int channels, long long samples, int bins, void* stream) {
  if (channels <= 0 || samples <= 0 || bins <= 0) return OA_ERR_ARG;
  audio_envelope_kernel<<<(bins + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, channels, samples, bins);
  return a_status();
}

}  // extern "C"
