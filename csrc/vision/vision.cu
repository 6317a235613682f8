// Image transforms, NeRF volume rendering, canvas painting and the fractional
// Grünwald–Letnikov stencil as plain CUDA compute on device buffers (no graphics API).
//
// Arithmetic restated from the reference's compute shaders:
//   * bilinear resize with half-pixel centres, centre crop, horizontal flip, colour jitter
//     (brightness → contrast around per-channel means → saturation → hue rotation in YUV)
//     — crates/st-backend-wgpu/shaders/transforms/{resize,center_crop,horizontal_flip,color_jitter}.wgsl;
//     plus `preprocess`: resize → crop → jitter → flip fused into ONE pass over the output;
//   * stratified ray samples and front-to-back compositing w = T·(1 − e^{−σδ}), rgb += w·c,
//     T *= 1 − α — crates/st-backend-wgpu/src/shaders/{nerf_volume_utils,nerf_raymarch}.wgsl;
//     the backward pass (dσ, dc) is new (the reference trains its NeRF on the CPU);
//   * palette painting of a tensor into RGBA8 — crates/st-tensor/src/pure/wasm_canvas.rs;
//   * y[i] = (Σ_{k ≤ min(i,m)} w[k]·x[i−k]) / h^α — crates/st-tensor/src/wgpu_shaders/frac_gl_1d.wgsl.
// Images are fp32 NCHW batches.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {

struct Jitter {
  float brightness, contrast, saturation, hue;  // factors; hue in radians
  float mean[4];                                // per-channel means used by the contrast step
};

__device__ __forceinline__ float bilinear(const float* __restrict__ img, int sh, int sw, float sy, float sx) {
  const float y0f = fminf(fmaxf(floorf(sy), 0.0f), (float)(sh - 1));
  const float x0f = fminf(fmaxf(floorf(sx), 0.0f), (float)(sw - 1));
  const int y0 = (int)y0f, x0 = (int)x0f;
  const int y1 = min(y0 + 1, sh - 1), x1 = min(x0 + 1, sw - 1);
  const float ly = sy - y0f, lx = sx - x0f;
  const float top = img[y0 * sw + x0] * (1.0f - lx) + img[y0 * sw + x1] * lx;
  const float bot = img[y1 * sw + x0] * (1.0f - lx) + img[y1 * sw + x1] * lx;
  return top * (1.0f - ly) + bot * ly;
}

__device__ __forceinline__ float bright_contrast(const Jitter& j, int c, float v) {
  const float b = v * j.brightness;
  if (j.contrast == 1.0f) return b;
  const float m = j.mean[min(c, 3)];
  return (b - m) * j.contrast + m;
}

__device__ __forceinline__ void jitter_rgb(const Jitter& j, float& r, float& g, float& b) {
  if (j.saturation != 1.0f) {
    const float gray = r * 0.29899597f + g * 0.587096f + b * 0.11390703f;
    r = (r - gray) * j.saturation + gray;
    g = (g - gray) * j.saturation + gray;
    b = (b - gray) * j.saturation + gray;
  }
  if (j.hue != 0.0f) {
    const float ch = cosf(j.hue), sh = sinf(j.hue);
    const float y = 0.299f * r + 0.587f * g + 0.114f * b;
    const float u = -0.14713f * r - 0.28886f * g + 0.436f * b;
    const float v = 0.615f * r - 0.51499f * g - 0.10001f * b;
    const float up = u * ch - v * sh, vp = u * sh + v * ch;
    r = y + 1.13983f * vp;
    g = y - 0.39465f * up - 0.58060f * vp;
    b = y + 2.03211f * up;
  }
}

// One thread per output pixel (all channels).  The pipeline is expressed as coordinate
// maps applied back to front: flip → crop offset → resize sample, then the colour math.
__global__ void preprocess_kernel(const float* __restrict__ in, float* __restrict__ out, int B, int C,
                                  int sh, int sw, int rh, int rw, int oh, int ow, int crop_y, int crop_x,
                                  int flip, Jitter jit, int do_jitter) {
  const long long total = (long long)B * oh * ow;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = i % ow;
    const int y = (i / ow) % oh;
    const int b = i / ((long long)ow * oh);
    const int xs = flip ? (ow - 1 - x) : x;
    const int ry = y + crop_y, rx = xs + crop_x;            // position in the resized image
    const float sy = (ry + 0.5f) * ((float)sh / rh) - 0.5f;
    const float sx = (rx + 0.5f) * ((float)sw / rw) - 0.5f;
    const float* img = in + (size_t)b * C * sh * sw;
    float px[4] = {0, 0, 0, 0};
    for (int c = 0; c < C; ++c) {
      float v = (rh == sh && rw == sw) ? img[(size_t)c * sh * sw + ry * sw + rx]
                                       : bilinear(img + (size_t)c * sh * sw, sh, sw, sy, sx);
      if (do_jitter) v = bright_contrast(jit, c, v);
      if (c < 4) px[c] = v;
      else out[((size_t)b * C + c) * oh * ow + (size_t)y * ow + x] = v;
    }
    if (do_jitter && C >= 3) jitter_rgb(jit, px[0], px[1], px[2]);
    for (int c = 0; c < min(C, 4); ++c) out[((size_t)b * C + c) * oh * ow + (size_t)y * ow + x] = px[c];
  }
}

// ---- NeRF ------------------------------------------------------------------------------------
__device__ __forceinline__ float lcg_offset(unsigned ray, unsigned sample, unsigned seed) {
  const unsigned base = ray * 9781u + seed * 6271u;
  const unsigned step = 1103515245u * (base + sample) + 12345u;
  return (float)((step >> 9) & 0x007fffffu) / (float)0x007fffff;
}

// rays: [R, 8] = origin(3), direction(3), t_min, t_max.  points: [R, S, 3], t: [R, S], deltas: [R, S].
__global__ void nerf_sample_kernel(const float* __restrict__ rays, float* __restrict__ points,
                                   float* __restrict__ ts, float* __restrict__ deltas, int R, int S,
                                   int stratified, unsigned seed) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const float* ray = rays + (size_t)r * 8;
  const float t_min = ray[6], t_max = ray[7];
  const float span = fmaxf(t_max - t_min, 1e-3f);
  const float interval = span / S;
  for (int i = 0; i < S; ++i) {
    const float off = stratified ? lcg_offset(r, i, seed) : 0.5f;
    const float t = t_min + (i + fminf(fmaxf(off, 0.0f), 0.999f)) * interval;
    const float next_t = (i + 1 == S) ? t_max : t_min + (i + 1) * interval;
    const size_t idx = (size_t)r * S + i;
    ts[idx] = t;
    deltas[idx] = fmaxf(next_t - t, 1e-3f);
    points[idx * 3 + 0] = ray[0] + ray[3] * t;
    points[idx * 3 + 1] = ray[1] + ray[4] * t;
    points[idx * 3 + 2] = ray[2] + ray[5] * t;
  }
}

// sigma: [R, S], radiance: [R, S, 3], deltas: [R, S]  ->  accum: [R, 4] = rgb, opacity.
__global__ void nerf_composite_fwd_kernel(const float* __restrict__ sigma, const float* __restrict__ rad,
                                          const float* __restrict__ deltas, float* __restrict__ accum,
                                          int R, int S, float delta_scale) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  float T = 1.0f, cr = 0.0f, cg = 0.0f, cb = 0.0f, op = 0.0f;
  for (int i = 0; i < S; ++i) {
    const size_t idx = (size_t)r * S + i;
    const float alpha = 1.0f - __expf(-fmaxf(sigma[idx], 0.0f) * deltas[idx] * delta_scale);
    const float w = T * alpha;
    cr += w * rad[idx * 3 + 0];
    cg += w * rad[idx * 3 + 1];
    cb += w * rad[idx * 3 + 2];
    op += w;
    T *= 1.0f - alpha;
  }
  accum[(size_t)r * 4 + 0] = cr;
  accum[(size_t)r * 4 + 1] = cg;
  accum[(size_t)r * 4 + 2] = cb;
  accum[(size_t)r * 4 + 3] = op;
}

// Backward of the compositing: given d(accum), produce d(sigma) and d(radiance).
// With suffix sums  S_i = Σ_{j>i} w_j (g·c_j + g_op):  dL/dα_i = T_i (g·c_i + g_op) − S_i / (1 − α_i).
__global__ void nerf_composite_bwd_kernel(const float* __restrict__ sigma, const float* __restrict__ rad,
                                          const float* __restrict__ deltas, const float* __restrict__ accum,
                                          const float* __restrict__ d_accum, float* __restrict__ d_sigma,
                                          float* __restrict__ d_rad, int R, int S, float delta_scale) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const float gr = d_accum[(size_t)r * 4], gg = d_accum[(size_t)r * 4 + 1], gb = d_accum[(size_t)r * 4 + 2],
              go = d_accum[(size_t)r * 4 + 3];
  // total = Σ_j w_j (g·c_j + go) is what the forward accumulated, projected on the gradient
  float remaining = gr * accum[(size_t)r * 4] + gg * accum[(size_t)r * 4 + 1] + gb * accum[(size_t)r * 4 + 2] +
                    go * accum[(size_t)r * 4 + 3];
  float T = 1.0f;
  for (int i = 0; i < S; ++i) {
    const size_t idx = (size_t)r * S + i;
    const float sg = sigma[idx];
    const float step = deltas[idx] * delta_scale;
    const float alpha = 1.0f - __expf(-fmaxf(sg, 0.0f) * step);
    const float w = T * alpha;
    const float dotc = gr * rad[idx * 3] + gg * rad[idx * 3 + 1] + gb * rad[idx * 3 + 2] + go;
    d_rad[idx * 3 + 0] = w * gr;
    d_rad[idx * 3 + 1] = w * gg;
    d_rad[idx * 3 + 2] = w * gb;
    remaining -= w * dotc;                                   // now the suffix sum over j > i
    const float one_m = fmaxf(1.0f - alpha, 1e-10f);
    const float d_alpha = T * dotc - remaining / one_m;
    d_sigma[idx] = sg > 0.0f ? d_alpha * step * (1.0f - alpha) : 0.0f;
    T *= 1.0f - alpha;
  }
}

// ---- canvas ------------------------------------------------------------------------------------
// palette 0: grayscale, 1: blue→magenta→yellow "spiral", 2: diverging blue/white/red
__global__ void canvas_paint_kernel(const float* __restrict__ x, unsigned char* __restrict__ rgba, long long n,
                                    float lo, float hi, int palette) {
  const float inv = hi > lo ? 1.0f / (hi - lo) : 0.0f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float t = (x[i] - lo) * inv;
    t = isfinite(t) ? fminf(fmaxf(t, 0.0f), 1.0f) : 0.0f;
    float r, g, b;
    if (palette == 0) {
      r = g = b = t;
    } else if (palette == 1) {
      r = fminf(1.0f, 1.6f * t);
      g = t * t;
      b = fminf(1.0f, 0.35f + 0.9f * (1.0f - fabsf(2.0f * t - 1.0f)));
    } else {
      r = t < 0.5f ? 2.0f * t : 1.0f;
      b = t < 0.5f ? 1.0f : 2.0f * (1.0f - t);
      g = 1.0f - fabsf(2.0f * t - 1.0f);
    }
    rgba[i * 4 + 0] = (unsigned char)(r * 255.0f + 0.5f);
    rgba[i * 4 + 1] = (unsigned char)(g * 255.0f + 0.5f);
    rgba[i * 4 + 2] = (unsigned char)(b * 255.0f + 0.5f);
    rgba[i * 4 + 3] = 255;
  }
}

// ---- fractional GL stencil ----------------------------------------------------------------------
__global__ void frac_gl_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                               int rows, int n, int m, float inv_h_alpha) {
  extern __shared__ float sw[];
  for (int k = threadIdx.x; k <= m; k += blockDim.x) sw[k] = w[k];
  __syncthreads();
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* xr = x + (size_t)row * n;
  const int kmax = min(i, m);
  float acc = 0.0f;
  for (int k = 0; k <= kmax; ++k) acc += sw[k] * xr[i - k];
  y[(size_t)row * n + i] = acc * inv_h_alpha;
}

inline int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)st::sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

struct StPreprocessArgs {
  int B, C, src_h, src_w, resize_h, resize_w, out_h, out_w, crop_y, crop_x, flip, do_jitter;
  float brightness, contrast, saturation, hue;
  float mean[4];
};

// out[b, c, y, x] for the pipeline resize(src → resize_h x resize_w) → crop(out_h x out_w at crop_y, crop_x)
// → colour jitter → horizontal flip.  Single transforms are special cases of the arguments.
ST_API int st_preprocess(const float* in, float* out, const StPreprocessArgs* a, void* stream_v) {
  if (!a || a->B <= 0 || a->C <= 0 || a->C > 16) return st::fail(ST_ERR_INVALID, "preprocess: bad batch/channels");
  if (a->crop_y < 0 || a->crop_x < 0 || a->crop_y + a->out_h > a->resize_h || a->crop_x + a->out_w > a->resize_w)
    return st::fail(ST_ERR_INVALID, "preprocess: crop window outside the resized image");
  Jitter j;
  j.brightness = a->brightness; j.contrast = a->contrast; j.saturation = a->saturation; j.hue = a->hue;
  for (int i = 0; i < 4; ++i) j.mean[i] = a->mean[i];
  const long long total = (long long)a->B * a->out_h * a->out_w;
  preprocess_kernel<<<grid_for(total, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      in, out, a->B, a->C, a->src_h, a->src_w, a->resize_h, a->resize_w, a->out_h, a->out_w, a->crop_y, a->crop_x,
      a->flip, j, a->do_jitter);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_nerf_sample(const float* rays, float* points, float* ts, float* deltas, int R, int S,
                          int stratified, unsigned seed, void* stream_v) {
  if (R <= 0 || S <= 0) return st::fail(ST_ERR_INVALID, "nerf_sample: empty problem");
  nerf_sample_kernel<<<(R + 63) / 64, 64, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(rays, points, ts, deltas,
                                                                                       R, S, stratified, seed);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_nerf_composite_fwd(const float* sigma, const float* rad, const float* deltas, float* accum, int R,
                                 int S, float delta_scale, void* stream_v) {
  if (R <= 0 || S <= 0) return st::fail(ST_ERR_INVALID, "nerf_composite: empty problem");
  nerf_composite_fwd_kernel<<<(R + 63) / 64, 64, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      sigma, rad, deltas, accum, R, S, delta_scale);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_nerf_composite_bwd(const float* sigma, const float* rad, const float* deltas, const float* accum,
                                 const float* d_accum, float* d_sigma, float* d_rad, int R, int S,
                                 float delta_scale, void* stream_v) {
  if (R <= 0 || S <= 0) return st::fail(ST_ERR_INVALID, "nerf_composite: empty problem");
  nerf_composite_bwd_kernel<<<(R + 63) / 64, 64, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      sigma, rad, deltas, accum, d_accum, d_sigma, d_rad, R, S, delta_scale);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_canvas_paint(const float* x, unsigned char* rgba, long long n, float lo, float hi, int palette,
                           void* stream_v) {
  if (n <= 0) return ST_OK;
  canvas_paint_kernel<<<grid_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(x, rgba, n, lo, hi,
                                                                                            palette);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_frac_gl(const float* x, const float* w, float* y, int rows, int n, int m, float h_alpha,
                      void* stream_v) {
  if (rows <= 0 || n <= 0 || m < 0) return st::fail(ST_ERR_INVALID, "frac_gl: empty problem");
  if (m > 8191) return st::fail(ST_ERR_TOO_LARGE, "frac_gl: at most 8192 stencil weights");
  if (!(h_alpha > 0.0f)) return st::fail(ST_ERR_INVALID, "frac_gl: h^alpha must be positive");
  dim3 grid((n + 255) / 256, rows);
  frac_gl_kernel<<<grid, 256, (m + 1) * sizeof(float), reinterpret_cast<cudaStream_t>(stream_v)>>>(
      x, w, y, rows, n, m, 1.0f / h_alpha);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
