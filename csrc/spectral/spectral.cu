// Spectral kernels: batched 1-D FFT in shared memory (any stride, real or complex input, optional window,
// power-of-two lengths by Stockham radix-8 passes with the butterflies in registers and other lengths by a direct
// DFT against a shared twiddle table), spectral multipliers for the fractional operators, and the temporal volume
// renderer.
//
// All of them are bandwidth-bound elementwise / small-transform work: one pass over the data, fp32 math,
// no tensor cores.  A transform lives entirely in one CTA's shared memory (two ping-pong buffers), so a batch
// of transforms costs one read and one write of the data whatever the length.
#include <cuda_runtime.h>
#include <cstdint>
#include <math_constants.h>

#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {

constexpr int kMaxFftLen = 8192;        // 2 x 8192 complex fp32 = 128 KB of shared memory
constexpr int kMaxDftLen = 4096;        // direct DFT: input + twiddle table
constexpr float kTau = 6.283185307179586f;
constexpr int kMaxRenderTableFrames = 4096;   // 32 KB of (sin, cos) per CTA
constexpr int kRenderRegChannels = 8;         // harmonic amplitudes kept in registers across the frame loop

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

// ---- in-register DFTs of 2, 4 and 8 points (forward sign, natural output order) -------------------------------
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ float2 mul_neg_i(float2 a) { return make_float2(a.y, -a.x); }          // a * (-i)

__device__ __forceinline__ void dft4(float2& x0, float2& x1, float2& x2, float2& x3) {
  const float2 a = cadd(x0, x2), b = csub(x0, x2), c = cadd(x1, x3), d = mul_neg_i(csub(x1, x3));
  x0 = cadd(a, c); x1 = cadd(b, d); x2 = csub(a, c); x3 = csub(b, d);
}

template <int R>
__device__ __forceinline__ void dft_regs(float2 (&v)[8]) {
  if constexpr (R == 2) {
    const float2 a = v[0];
    v[0] = cadd(a, v[1]); v[1] = csub(a, v[1]);
  } else if constexpr (R == 4) {
    dft4(v[0], v[1], v[2], v[3]);
  } else {
    float2 e0 = v[0], e1 = v[2], e2 = v[4], e3 = v[6], o0 = v[1], o1 = v[3], o2 = v[5], o3 = v[7];
    dft4(e0, e1, e2, e3);
    dft4(o0, o1, o2, o3);
    constexpr float h = 0.70710678118654752f;
    o1 = make_float2(h * (o1.x + o1.y), h * (o1.y - o1.x));            // * exp(-i pi / 4)
    o2 = mul_neg_i(o2);                                                 // * exp(-i pi / 2)
    o3 = make_float2(h * (o3.y - o3.x), -h * (o3.x + o3.y));           // * exp(-3 i pi / 4)
    v[0] = cadd(e0, o0); v[4] = csub(e0, o0);
    v[1] = cadd(e1, o1); v[5] = csub(e1, o1);
    v[2] = cadd(e2, o2); v[6] = csub(e2, o2);
    v[3] = cadd(e3, o3); v[7] = csub(e3, o3);
  }
}

// Shared-memory slot of point i: 8 slots of padding per 64 points (the second pass writes groups of 8 consecutive
// points that are 64 points apart) and the low three bits XOR-ed with bits 4..6 of i (the first pass writes 8
// consecutive points per thread, so 16 threads of a half-warp would land on two bank pairs without it).  With both,
// every 64-bit shared-memory access of every pass touches 16 distinct bank pairs per half-warp.
__device__ __forceinline__ int slot(int i) { return (i + ((i >> 6) << 3)) ^ ((i >> 4) & 7); }

// One Stockham pass of radix R over a transform of n points whose sub-transforms already have length ns:
//   v[r] = src[j + r n/R] * w^r (w = exp(-2 pi i (j mod ns) / (ns R))), DFT_R(v), dst[(j / ns) ns R + (j mod ns) + r ns] = v[r]
// FIRST reads the (strided, possibly real, windowed) input from global memory, LAST writes the output there, so a
// transform of three passes crosses shared memory twice.  The inverse transform is conj(FFT(conj(x))) / n.
// NSC is ns when it is 1, 8 or 64 and 0 for a run-time ns that is a multiple of 512: each case has a closed form of
// slot() for its eight outputs (one XOR and one add per output instead of the shifts of the general formula).
// VEC: input and output are interleaved complex with unit stride, moved as float2.
template <int R, bool FIRST, bool LAST, int NSC, bool VEC>
__device__ __forceinline__ void stockham_pass(const float2* __restrict__ src, float2* __restrict__ dst, const float* __restrict__ gin,
                                              float* __restrict__ gout, const float* __restrict__ window, long long in_i,
                                              long long out_i, int n, int ns_rt, int complex_in, int inverse, float scale) {
  const int ns = NSC ? NSC : ns_rt;
  const int m = n / R;
  const bool stride_reads = (m & 127) == 0;          // slot(j + r m) = slot(j) + r (m + m / 8)
  const int m_slots = m + (m >> 3);
  const float angle_scale = -2.0f / (float)(ns * R);  // a power of two: exact
  for (int j = threadIdx.x; j < m; j += blockDim.x) {
    float2 v[8];
    if constexpr (FIRST) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = j + r * m;
        const float w = window ? window[i] : 1.0f;
        float re, im;
        if constexpr (VEC) {
          const float2 x = reinterpret_cast<const float2*>(gin)[i];
          re = x.x; im = x.y;
        } else {
          re = gin[i * in_i];
          im = complex_in ? gin[i * in_i + 1] : 0.0f;
        }
        v[r] = make_float2(re * w, inverse ? -im * w : im * w);
      }
    } else {
      const int s0 = slot(j);
#pragma unroll
      for (int r = 0; r < R; ++r) v[r] = src[stride_reads ? s0 + r * m_slots : slot(j + r * m)];
    }
    const int k = j & (ns - 1);
    if constexpr (!FIRST) {
      float sn, cs;
      sincospif((float)k * angle_scale, &sn, &cs);
      const float2 w1 = make_float2(cs, sn);
      v[1] = cmul(v[1], w1);
      if constexpr (R >= 4) {
        const float2 w2 = cmul(w1, w1), w3 = cmul(w2, w1);
        v[2] = cmul(v[2], w2); v[3] = cmul(v[3], w3);
        if constexpr (R == 8) {
          const float2 w4 = cmul(w2, w2);
          v[4] = cmul(v[4], w4); v[5] = cmul(v[5], cmul(w4, w1)); v[6] = cmul(v[6], cmul(w4, w2)); v[7] = cmul(v[7], cmul(w4, w3));
        }
      }
    }
    dft_regs<R>(v);
    if constexpr (LAST) {
      const int j0 = (j - k) * R + k;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int o = j0 + r * ns;
        const float2 y = make_float2(v[r].x * scale, (inverse ? -v[r].y : v[r].y) * scale);
        if constexpr (VEC) {
          reinterpret_cast<float2*>(gout)[o] = y;
        } else {
          gout[o * out_i] = y.x;
          gout[o * out_i + 1] = y.y;
        }
      }
    } else {
      static_assert(LAST || R == 8, "only radix-8 passes write shared memory");
      if constexpr (NSC == 1) {
        const int base = j * 8 + ((j >> 3) << 3), x = (j >> 1) & 7;
#pragma unroll
        for (int r = 0; r < 8; ++r) dst[base + (r ^ x)] = v[r];
      } else if constexpr (NSC == 8) {
        const int g = j >> 3, base = g * 72, x = k ^ ((g & 1) << 2);
#pragma unroll
        for (int r = 0; r < 8; ++r) dst[base + r * 8 + (x ^ (r >> 1))] = v[r];
      } else if constexpr (NSC == 64) {
        const int base = (j >> 6) * 576, x = k ^ (k >> 4);
#pragma unroll
        for (int r = 0; r < 8; ++r) dst[base + r * 72 + (x ^ ((r & 1) << 2))] = v[r];
      } else {
        const int ns_slots = ns + (ns >> 3);
        const int base = ((j - k) / ns) * 8 * ns_slots + slot(k);
#pragma unroll
        for (int r = 0; r < 8; ++r) dst[base + r * ns_slots] = v[r];
      }
    }
  }
}

// One transform per CTA: n = 8^a * tail with tail in {1, 2, 4}; `a` radix-8 passes, then the tail pass.
template <bool VEC>
__global__ void __launch_bounds__(512, 2)
fft_pow2_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ window,
                FftLayout L, int n, int log2n, int complex_in, int inverse) {
  extern __shared__ float2 smem[];
  const int padded = n + (((n - 1) >> 6) << 3);
  float2* a = smem;
  float2* b = smem + padded;
  const int batch = blockIdx.x;
  const int b0 = batch / L.batch1, b1 = batch % L.batch1;
  const float* gin = in + b0 * L.in_b0 + b1 * L.in_b1;
  float* gout = out + b0 * L.out_b0 + b1 * L.out_b1;
  const float scale = inverse ? 1.0f / (float)n : 1.0f;
  const int eights = log2n / 3, tail = 1 << (log2n - 3 * eights);
#define ST_FFT_PASS(R, FIRST, LAST, NSC, SRC, DST, NS) \
  stockham_pass<R, FIRST, LAST, NSC, VEC>(SRC, DST, gin, gout, window, L.in_i, L.out_i, n, NS, complex_in, inverse, scale)
  if (n == 1) {
    if (threadIdx.x == 0) {
      const float w = window ? window[0] : 1.0f;
      gout[0] = gin[0] * w;
      gout[1] = complex_in ? gin[1] * w : 0.0f;
    }
    return;
  }
  if (eights == 0) {               // n = 2 or 4: a single pass from global to global
    if (tail == 2) ST_FFT_PASS(2, true, true, 1, nullptr, nullptr, 1);
    else ST_FFT_PASS(4, true, true, 1, nullptr, nullptr, 1);
    return;
  }
  if (eights == 1 && tail == 1) {  // n = 8
    ST_FFT_PASS(8, true, true, 1, nullptr, nullptr, 1);
    return;
  }
  ST_FFT_PASS(8, true, false, 1, nullptr, a, 1);
  __syncthreads();
  float2* src = a;
  float2* dst = b;
  int ns = 8;
  for (int p = 1; p < eights; ++p) {
    if (p == eights - 1 && tail == 1) {
      if (p == 1) ST_FFT_PASS(8, false, true, 8, src, nullptr, 8);
      else if (p == 2) ST_FFT_PASS(8, false, true, 64, src, nullptr, 64);
      else ST_FFT_PASS(8, false, true, 0, src, nullptr, ns);
      return;
    }
    if (p == 1) ST_FFT_PASS(8, false, false, 8, src, dst, 8);
    else if (p == 2) ST_FFT_PASS(8, false, false, 64, src, dst, 64);
    else ST_FFT_PASS(8, false, false, 0, src, dst, ns);
    __syncthreads();
    float2* t = src; src = dst; dst = t;
    ns *= 8;
  }
  if (tail == 2) ST_FFT_PASS(2, false, true, 0, src, nullptr, ns);
  else ST_FFT_PASS(4, false, true, 0, src, nullptr, ns);
#undef ST_FFT_PASS
}

// Streaming form for long batches of contiguous complex rows: a persistent CTA walks rows blockIdx.x, + gridDim.x, ...
// and, while it works through the passes of one row, a bulk asynchronous copy brings the next row into a staging
// buffer, so the only exposed global-memory latency is that of the CTA's first row.  The first pass reads the staging
// buffer; everything else is the kernel above.  n = 8^a * tail with a >= 2.
__global__ void __launch_bounds__(512, 2)
fft_pow2_stream_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ window,
                       FftLayout L, int n, int log2n, int inverse, int batches, unsigned* err) {
  extern __shared__ __align__(16) float2 smem[];
  constexpr bool VEC = true;
  constexpr int complex_in = 1;
  const int padded = n + (((n - 1) >> 6) << 3);
  float2* a = smem;
  float2* b = smem + padded;
  float2* stage = smem + 2 * padded;                                  // n complex values, 16-byte aligned (padded is a multiple of 8)
  uint64_t* bar = reinterpret_cast<uint64_t*>(stage + n);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);
  const uint32_t row_bytes = static_cast<uint32_t>(n) * 8u;
  auto row_in = [&](int batch) { return in + (batch / L.batch1) * L.in_b0 + (batch % L.batch1) * L.in_b1; };
  if (threadIdx.x == 0) {
    st::mbar_init(st::smem_u32(bar), 1);
    *abort_flag = 0;
    st::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < batches) {
    st::mbar_arrive_expect_tx(st::smem_u32(bar), row_bytes);
    st::bulk_load_g2s(st::smem_u32(stage), row_in(blockIdx.x), row_bytes, st::smem_u32(bar));
  }
  const float scale = inverse ? 1.0f / (float)n : 1.0f;
  const int eights = log2n / 3, tail = 1 << (log2n - 3 * eights);
  uint32_t phase = 0;
  for (int batch = blockIdx.x; batch < batches; batch += gridDim.x) {
    float* gout = out + (batch / L.batch1) * L.out_b0 + (batch % L.batch1) * L.out_b1;
    const float* gin = reinterpret_cast<const float*>(stage);
    // bounded wait; the CTA decides together, so nobody is left at a barrier by a thread that gave up
    if (!__syncthreads_and(st::mbar_wait(st::smem_u32(bar), phase, abort_flag) ? 1 : 0)) break;
    phase ^= 1u;
#define ST_FFT_PASS(R, FIRST, LAST, NSC, SRC, DST, NS) \
  stockham_pass<R, FIRST, LAST, NSC, VEC>(SRC, DST, gin, gout, window, L.in_i, L.out_i, n, NS, complex_in, inverse, scale)
    ST_FFT_PASS(8, true, false, 1, nullptr, a, 1);
    __syncthreads();                       // the staging buffer has been read by everyone: refill it with the next row
    if (threadIdx.x == 0 && batch + static_cast<int>(gridDim.x) < batches) {
      st::mbar_arrive_expect_tx(st::smem_u32(bar), row_bytes);
      st::bulk_load_g2s(st::smem_u32(stage), row_in(batch + gridDim.x), row_bytes, st::smem_u32(bar));
    }
    float2* src = a;
    float2* dst = b;
    int ns = 8;
    bool done = false;
    for (int p = 1; p < eights && !done; ++p) {
      if (p == eights - 1 && tail == 1) {
        if (p == 1) ST_FFT_PASS(8, false, true, 8, src, nullptr, 8);
        else if (p == 2) ST_FFT_PASS(8, false, true, 64, src, nullptr, 64);
        else ST_FFT_PASS(8, false, true, 0, src, nullptr, ns);
        done = true;
        break;
      }
      if (p == 1) ST_FFT_PASS(8, false, false, 8, src, dst, 8);
      else if (p == 2) ST_FFT_PASS(8, false, false, 64, src, dst, 64);
      else ST_FFT_PASS(8, false, false, 0, src, dst, ns);
      __syncthreads();
      float2* t = src; src = dst; dst = t;
      ns *= 8;
    }
    if (!done) {
      if (tail == 2) ST_FFT_PASS(2, false, true, 0, src, nullptr, ns);
      else ST_FFT_PASS(4, false, true, 0, src, nullptr, ns);
    }
#undef ST_FFT_PASS
    __syncthreads();                       // the last pass has read its source before the next row's first pass writes `a`
  }
  if (*abort_flag && threadIdx.x == 0) st::report_error(err, st::ERR_MBAR_TIMEOUT, 0xF7F1u);
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
// One thread owns a column: the multiplier (a pow and, for the derivative, a sincos) is computed once and applied to
// that column of `rows_per_block` consecutive rows, so the kernel is a streaming multiply.
__global__ void specmul_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int cols, float power,
                               float inv_h, int mode, int rows_per_block) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float2 mult;
  bool passthrough = false, infinite = false;
  if (mode == 0) {
    const int mirror = cols - 1 - col;
    mult = make_float2(powf(fmaxf((float)(col < mirror ? col : mirror), 0.0f), power), 0.0f);
  } else {
    const int k = col < (cols + 1) / 2 ? col : col - cols;      // fftfreq ordering
    const float omega = kTau * (float)k * inv_h / (float)cols;
    if (k == 0) {
      mult = make_float2(0.0f, 0.0f);
      passthrough = power == 0.0f;
      infinite = power < 0.0f;
    } else {
      // (i omega)^a = |omega|^a * exp(i * a * sign(omega) * pi / 2)
      const float mag = powf(fabsf(omega), power);
      float sn, cs;
      sincosf(power * (omega > 0.0f ? 1.0f : -1.0f) * 1.5707963267948966f, &sn, &cs);
      mult = make_float2(mag * cs, mag * sn);
    }
  }
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  const float2* xp = reinterpret_cast<const float2*>(x);
  float2* yp = reinterpret_cast<float2*>(y);
#pragma unroll 4
  for (long long r = r0; r < r1; ++r) {
    const float2 v = xp[r * cols + col];
    yp[r * cols + col] = passthrough ? v : (infinite ? make_float2(CUDART_INF_F, CUDART_INF_F) : cmul(v, mult));
  }
}

// out[f, v] = (voxel[v] + sum_c harm[v, c] * sin((c + 1) * tau * t_f)) * exp(-decay[v] * t_f), t_f = f / rate.
// decay: non-finite -> 1, negative -> 0; decay <= eps gives 0.  sin((c+1) theta) advances by the Chebyshev
// recurrence s_{c+1} = 2 cos(theta) s_c - s_{c-1}, so a frame costs one sincos per voxel however many channels.
__global__ void temporal_render_kernel(const float* __restrict__ voxels, const float* __restrict__ harmonics,
                                       const float* __restrict__ decay, float* __restrict__ out, long long n_voxels,
                                       int channels, int frames, float dt) {
  // sin / cos of the base angle of every frame are the same for all voxels: one table per CTA
  extern __shared__ float2 frame_sc[];
  const bool table = channels > 0 && frames <= kMaxRenderTableFrames;
  if (table) {
    for (int f = threadIdx.x; f < frames; f += blockDim.x) {
      float sn, cs;
      sincosf(kTau * ((float)f * dt), &sn, &cs);
      frame_sc[f] = make_float2(sn, cs);
    }
    __syncthreads();
  }
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < n_voxels;
       v += (long long)gridDim.x * blockDim.x) {
    const float base0 = voxels[v];
    float d = decay[v];
    d = isfinite(d) ? fmaxf(d, 0.0f) : 1.0f;
    const float* h = harmonics + v * channels;
    float amp[kRenderRegChannels];
    const bool in_regs = channels <= kRenderRegChannels;
    if (in_regs) {
#pragma unroll
      for (int c = 0; c < kRenderRegChannels; ++c) amp[c] = c < channels ? h[c] : 0.0f;
    }
    for (int f = 0; f < frames; ++f) {
      const float t = (float)f * dt;
      float base = base0;
      if (channels > 0) {
        float sn, cs;
        if (table) { sn = frame_sc[f].x; cs = frame_sc[f].y; } else { sincosf(kTau * t, &sn, &cs); }
        float s_prev = 0.0f, s_cur = sn;                 // sin(0 * theta), sin(1 * theta)
        const float two_c = 2.0f * cs;
        if (in_regs) {
#pragma unroll
          for (int c = 0; c < kRenderRegChannels; ++c) {
            if (fabsf(amp[c]) > 1.1920929e-07f) base += amp[c] * s_cur;
            const float s_next = two_c * s_cur - s_prev;
            s_prev = s_cur; s_cur = s_next;
          }
        } else {
          for (int c = 0; c < channels; ++c) {
            const float a = h[c];
            if (fabsf(a) > 1.1920929e-07f) base += a * s_cur;
            const float s_next = two_c * s_cur - s_prev;
            s_prev = s_cur; s_cur = s_next;
          }
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
  const size_t padded = (size_t)a->n + (((size_t)a->n - 1) >> 6 << 3);          // 8 slots of padding per 64 points, as slot() in the kernel
  const size_t smem = pow2 ? 2 * padded * sizeof(float2) : 2 * (size_t)a->n * sizeof(float2);
  static bool configured[st::kMaxDevices][2] = {};
  const int dev = st::current_device();
  if (pow2) {
    if (smem > 48 * 1024 && !configured[dev][0]) {
      const int max_smem = 2 * (kMaxFftLen + kMaxFftLen / 8) * (int)sizeof(float2);
      ST_CUDA_CHECK(cudaFuncSetAttribute(fft_pow2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      ST_CUDA_CHECK(cudaFuncSetAttribute(fft_pow2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
      configured[dev][0] = true;
    }
    int log2n = 0;
    while ((1 << log2n) < a->n) ++log2n;
    int threads = a->n / 8;                    // one radix-8 butterfly per thread and pass
    threads = threads < 32 ? 32 : (threads > 512 ? 512 : threads);
    // interleaved complex on both sides with unit stride and 8-byte aligned transforms: float2 loads and stores
    const bool vec = a->complex_in && a->in_i == 2 && a->out_i == 2 && a->n > 1 &&
                     ((a->in_b0 | a->in_b1 | a->out_b0 | a->out_b1) & 1) == 0 &&
                     ((reinterpret_cast<uintptr_t>(a->in) | reinterpret_cast<uintptr_t>(a->out)) & 7) == 0;
    // long batches of contiguous, 16-byte aligned rows: persistent CTAs with the next row prefetched asynchronously
    const size_t stream_smem = smem + (size_t)a->n * sizeof(float2) + 16;
    const bool streamed = vec && log2n >= 6 && a->n <= 4096 && grid > 4 * st::sm_count() &&
                          ((a->in_b0 | a->in_b1) & 3) == 0 && (reinterpret_cast<uintptr_t>(a->in) & 15) == 0;
    if (streamed) {
      static bool stream_cfg[st::kMaxDevices] = {};
      if (!stream_cfg[dev]) {
        ST_CUDA_CHECK(cudaFuncSetAttribute(fft_pow2_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (2 * (4096 + 4096 / 8) + 4096) * (int)sizeof(float2) + 16));
        stream_cfg[dev] = true;
      }
      fft_pow2_stream_kernel<<<2 * st::sm_count(), threads, stream_smem, stream>>>(a->in, a->out, a->window, L, a->n, log2n, a->inverse,
                                                                                    grid, st::error_word());
    } else if (vec) fft_pow2_kernel<true><<<grid, threads, smem, stream>>>(a->in, a->out, a->window, L, a->n, log2n, a->complex_in, a->inverse);
    else fft_pow2_kernel<false><<<grid, threads, smem, stream>>>(a->in, a->out, a->window, L, a->n, log2n, a->complex_in, a->inverse);
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
  const int threads = cols >= 128 ? 128 : 32;
  const int col_blocks = (cols + threads - 1) / threads;
  // enough row chunks to fill the machine a few times over, each long enough to amortise the multiplier
  long long chunks = ((long long)st::sm_count() * 16 + col_blocks - 1) / col_blocks;
  if (chunks > rows) chunks = rows;
  if (chunks > 65535) chunks = 65535;
  if (chunks < 1) chunks = 1;
  const long long rows_per_block = (rows + chunks - 1) / chunks;
  if (rows_per_block > 2147483647LL) return st::fail(ST_ERR_TOO_LARGE, "specmul: too many rows");
  chunks = (rows + rows_per_block - 1) / rows_per_block;
  specmul_kernel<<<dim3(col_blocks, (unsigned)chunks), threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      x_reim, y_reim, rows, cols, power, mode == 1 ? 1.0f / h : 0.0f, mode, (int)rows_per_block);
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
  const size_t table = (channels > 0 && frames <= kMaxRenderTableFrames) ? (size_t)frames * sizeof(float2) : 0;
  temporal_render_kernel<<<(int)blocks, 256, table, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      voxels, harmonics, decay, out, n_voxels, channels, frames, 1.0f / sample_rate_hz);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
