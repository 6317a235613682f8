// Spectral kernels: batched 1-D FFT in shared memory (any stride, real or complex input, optional window,
// power-of-two lengths by Stockham radix-2 passes and other lengths by a direct DFT against a shared twiddle
// table), spectral multipliers for the fractional operators, and the temporal volume renderer.
//
// All of them are bandwidth-bound elementwise / small-transform work: one pass over the data, fp32 math,
// no tensor cores.  A transform lives entirely in one CTA's shared memory (two ping-pong buffers), so a batch
// of transforms costs one read and one write of the data whatever the length.
#include <cuda_runtime.h>
#include <math_constants.h>

#include "../common/host.h"

namespace {

constexpr int kMaxFftLen = 8192;        // 2 x 8192 complex fp32 = 128 KB of shared memory
constexpr int kMaxDftLen = 4096;        // direct DFT: input + twiddle table
constexpr float kTau = 6.283185307179586f;

struct FftLayout {
  // element (b0, b1, i) of the input lives at in[b0 * in_b0 + b1 * in_b1 + i * in_i] (in floats; complex input
  // has its imaginary part at +1); the output, always interleaved complex, at out[b0 * out_b0 + b1 * out_b1 + i * out_i]
  long long in_b0, in_b1, in_i;
  long long out_b0, out_b1, out_i;
  int batch1;                           // batches are numbered b = b0 * batch1 + b1
};

__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}

// One transform per CTA.  Stockham autosort: pass s (half = 1, 2, 4, ...) reads x[j + k*half] style pairs from
// `src` and writes in natural order to `dst`, so no bit-reversal pass is needed.
__global__ void fft_pow2_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ window,
                                FftLayout L, int n, int log2n, int complex_in, int inverse) {
  extern __shared__ float2 smem[];
  float2* a = smem;
  float2* b = smem + n;
  const int batch = blockIdx.x;
  const int b0 = batch / L.batch1, b1 = batch % L.batch1;
  const float* src_ptr = in + b0 * L.in_b0 + b1 * L.in_b1;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float w = window ? window[i] : 1.0f;
    const float re = src_ptr[i * L.in_i];
    const float im = complex_in ? src_ptr[i * L.in_i + 1] : 0.0f;
    a[i] = make_float2(re * w, im * w);
  }
  __syncthreads();
  const float sign = inverse ? 1.0f : -1.0f;
  const int half_n = n >> 1;
  // Stockham: at stage with `l` = number of already-combined points per group (1, 2, 4, ...) and m = n / (2l)
  // groups: y[j*2l + k] = x[j*l + k] + w * x[j*l + k + n/2], y[j*2l + k + l] = x[...] - w * x[...]
  float2* src = a;
  float2* dst = b;
  for (int l = 1; l < n; l <<= 1) {
    for (int t = threadIdx.x; t < half_n; t += blockDim.x) {
      const int k = t & (l - 1);          // position inside the group
      const int j = t / l;                // group index
      float sn, cs;
      sincospif(sign * (float)k / (float)l, &sn, &cs);          // exp(sign * 2 pi i k / 2l)
      const float2 w = make_float2(cs, sn);
      const float2 u = src[j * l + k];
      const float2 v = cmul(w, src[j * l + k + half_n]);
      dst[j * 2 * l + k] = make_float2(u.x + v.x, u.y + v.y);
      dst[j * 2 * l + k + l] = make_float2(u.x - v.x, u.y - v.y);
    }
    __syncthreads();
    float2* tmp = src; src = dst; dst = tmp;
  }
  const float scale = inverse ? 1.0f / (float)n : 1.0f;
  float* dst_ptr = out + b0 * L.out_b0 + b1 * L.out_b1;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float2 v = src[i];
    dst_ptr[i * L.out_i] = v.x * scale;
    dst_ptr[i * L.out_i + 1] = v.y * scale;
  }
  (void)log2n;
}

// Direct DFT for lengths that are not powers of two: out[k] = sum_i x[i] * w^(k*i mod n), twiddles from a table.
__global__ void dft_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ window,
                           FftLayout L, int n, int complex_in, int inverse) {
  extern __shared__ float2 smem[];
  float2* x = smem;
  float2* tw = smem + n;
  const int batch = blockIdx.x;
  const int b0 = batch / L.batch1, b1 = batch % L.batch1;
  const float* src_ptr = in + b0 * L.in_b0 + b1 * L.in_b1;
  const float sign = inverse ? 1.0f : -1.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float w = window ? window[i] : 1.0f;
    x[i] = make_float2(src_ptr[i * L.in_i] * w, complex_in ? src_ptr[i * L.in_i + 1] * w : 0.0f);
    float sn, cs;
    sincospif(sign * 2.0f * (float)i / (float)n, &sn, &cs);
    tw[i] = make_float2(cs, sn);
  }
  __syncthreads();
  const float scale = inverse ? 1.0f / (float)n : 1.0f;
  float* dst_ptr = out + b0 * L.out_b0 + b1 * L.out_b1;
  for (int k = threadIdx.x; k < n; k += blockDim.x) {
    float2 acc = make_float2(0.0f, 0.0f);
    int idx = 0;                                    // k * i mod n, advanced incrementally
    for (int i = 0; i < n; ++i) {
      const float2 p = cmul(x[i], tw[idx]);
      acc.x += p.x; acc.y += p.y;
      idx += k;
      if (idx >= n) idx -= n;
    }
    dst_ptr[k * L.out_i] = acc.x * scale;
    dst_ptr[k * L.out_i + 1] = acc.y * scale;
  }
}

// mode 0: fractional-Laplacian envelope, scale = min(col, cols - 1 - col)^power (real multiplier)
// mode 1: fractional derivative, multiplier = (i * omega_col)^alpha with omega = 2 pi * fftfreq(cols, h);
//         the zero frequency is set to 0 for alpha > 0
__global__ void specmul_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int cols, float power,
                               float inv_h, int mode) {
  const long long total = rows * cols;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(idx % cols);
    const float2 v = reinterpret_cast<const float2*>(x)[idx];
    float2 r;
    if (mode == 0) {
      const int mirror = cols - 1 - col;
      const float s = powf(fmaxf((float)(col < mirror ? col : mirror), 0.0f), power);
      r = make_float2(v.x * s, v.y * s);
    } else {
      const int k = col < (cols + 1) / 2 ? col : col - cols;      // fftfreq ordering
      const float omega = kTau * (float)k * inv_h / (float)cols;
      if (k == 0) {
        r = power > 0.0f ? make_float2(0.0f, 0.0f) : (power == 0.0f ? v : make_float2(CUDART_INF_F, CUDART_INF_F));
      } else {
        // (i omega)^a = |omega|^a * exp(i * a * sign(omega) * pi / 2)
        const float mag = powf(fabsf(omega), power);
        float sn, cs;
        sincosf(power * (omega > 0.0f ? 1.0f : -1.0f) * 1.5707963267948966f, &sn, &cs);
        r = cmul(v, make_float2(mag * cs, mag * sn));
      }
    }
    reinterpret_cast<float2*>(y)[idx] = r;
  }
}

// out[f, v] = (voxel[v] + sum_c harm[v, c] * sin((c + 1) * tau * t_f)) * exp(-decay[v] * t_f), t_f = f / rate.
// decay: non-finite -> 1, negative -> 0; decay <= eps gives 0.  sin((c+1) theta) advances by the Chebyshev
// recurrence s_{c+1} = 2 cos(theta) s_c - s_{c-1}, so a frame costs one sincos per voxel however many channels.
__global__ void temporal_render_kernel(const float* __restrict__ voxels, const float* __restrict__ harmonics,
                                       const float* __restrict__ decay, float* __restrict__ out, long long n_voxels,
                                       int channels, int frames, float dt) {
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < n_voxels;
       v += (long long)gridDim.x * blockDim.x) {
    const float base0 = voxels[v];
    float d = decay[v];
    d = isfinite(d) ? fmaxf(d, 0.0f) : 1.0f;
    const float* h = harmonics + v * channels;
    for (int f = 0; f < frames; ++f) {
      const float t = (float)f * dt;
      float base = base0;
      if (channels > 0) {
        float sn, cs;
        sincosf(kTau * t, &sn, &cs);
        float s_prev = 0.0f, s_cur = sn;                 // sin(0 * theta), sin(1 * theta)
        const float two_c = 2.0f * cs;
        for (int c = 0; c < channels; ++c) {
          const float amp = h[c];
          if (fabsf(amp) > 1.1920929e-07f) base += amp * s_cur;
          const float s_next = two_c * s_cur - s_prev;
          s_prev = s_cur; s_cur = s_next;
        }
      }
      out[(long long)f * n_voxels + v] = d <= 1.1920929e-07f ? 0.0f : base * __expf(-d * t);
    }
  }
}

}  // namespace

struct StFftArgs {
  const float* in;
  float* out;
  const float* window;     // n coefficients or null
  long long in_b0, in_b1, in_i, out_b0, out_b1, out_i;
  int n, batch0, batch1, complex_in, inverse;
};

ST_API int st_fft_max_len() { return kMaxFftLen; }
ST_API int st_dft_max_len() { return kMaxDftLen; }

ST_API int st_fft_1d(const StFftArgs* a, void* stream_v) {
  if (!a || !a->in || !a->out) return st::fail(ST_ERR_INVALID, "fft_1d: null argument");
  if (a->n <= 0 || a->batch0 <= 0 || a->batch1 <= 0) return st::fail(ST_ERR_INVALID, "fft_1d: empty problem");
  if ((long long)a->batch0 * a->batch1 > 2147483647LL) return st::fail(ST_ERR_TOO_LARGE, "fft_1d: too many transforms");
  const bool pow2 = (a->n & (a->n - 1)) == 0;
  if (pow2 ? a->n > kMaxFftLen : a->n > kMaxDftLen)
    return st::fail(ST_ERR_TOO_LARGE, "fft_1d: length above the shared-memory capacity (8192 power-of-two, 4096 other)");
  FftLayout L{a->in_b0, a->in_b1, a->in_i, a->out_b0, a->out_b1, a->out_i, a->batch1};
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int grid = a->batch0 * a->batch1;
  const size_t smem = 2 * (size_t)a->n * sizeof(float2);
  static bool configured[st::kMaxDevices][2] = {};
  const int dev = st::current_device();
  if (pow2) {
    if (smem > 48 * 1024 && !configured[dev][0]) {
      ST_CUDA_CHECK(cudaFuncSetAttribute(fft_pow2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kMaxFftLen * (int)sizeof(float2)));
      configured[dev][0] = true;
    }
    int log2n = 0;
    while ((1 << log2n) < a->n) ++log2n;
    const int threads = a->n >= 2048 ? 512 : (a->n >= 256 ? 128 : 32);
    fft_pow2_kernel<<<grid, threads, smem, stream>>>(a->in, a->out, a->window, L, a->n, log2n, a->complex_in, a->inverse);
  } else {
    if (smem > 48 * 1024 && !configured[dev][1]) {
      ST_CUDA_CHECK(cudaFuncSetAttribute(dft_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kMaxDftLen * (int)sizeof(float2)));
      configured[dev][1] = true;
    }
    const int threads = a->n >= 512 ? 256 : 64;
    dft_kernel<<<grid, threads, smem, stream>>>(a->in, a->out, a->window, L, a->n, a->complex_in, a->inverse);
  }
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_specmul(const float* x_reim, float* y_reim, long long rows, int cols, float power, float h, int mode,
                      void* stream_v) {
  if (rows <= 0 || cols <= 0) return st::fail(ST_ERR_INVALID, "specmul: empty problem");
  if (mode != 0 && mode != 1) return st::fail(ST_ERR_INVALID, "specmul: mode is 0 (Laplace envelope) or 1 (derivative)");
  if (!isfinite(power)) return st::fail(ST_ERR_INVALID, "specmul: power must be finite");
  if (mode == 1 && !(h > 0.0f)) return st::fail(ST_ERR_INVALID, "specmul: sample spacing must be positive");
  const long long total = rows * cols;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)st::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  specmul_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(x_reim, y_reim, rows, cols, power,
                                                                                   mode == 1 ? 1.0f / h : 0.0f, mode);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_temporal_render(const float* voxels, const float* harmonics, const float* decay, float* out,
                              long long n_voxels, int channels, int frames, float sample_rate_hz, void* stream_v) {
  if (n_voxels <= 0) return st::fail(ST_ERR_INVALID, "temporal_render: empty volume");
  if (frames <= 0) return st::fail(ST_ERR_INVALID, "temporal_render: needs at least one frame");
  if (!(sample_rate_hz > 0.0f) || !isfinite(sample_rate_hz)) return st::fail(ST_ERR_INVALID, "temporal_render: sample rate must be positive and finite");
  if (channels < 0 || (channels > 0 && !harmonics)) return st::fail(ST_ERR_INVALID, "temporal_render: harmonic buffer missing");
  long long blocks = (n_voxels + 255) / 256;
  const long long cap = (long long)st::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  temporal_render_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      voxels, harmonics, decay, out, n_voxels, channels, frames, 1.0f / sample_rate_hz);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
