// Fused optimizer steps on flat parameter buffers.
//
//   * AdamW with fp32 master weights, fp32 moments and bf16 working weights: one pass
//     reads grad/master/m/v and writes master/m/v/bf16-weight; the gradient scale
//     (1/accumulation steps x global-norm clip coefficient) is a device scalar so no host
//     synchronisation sits between backward and the step; optionally zeroes the gradient.
//   * SGD with momentum, same layout.
//   * sum of squares of a flat gradient (for the global norm) and the clip coefficient.
//   * Amegagrad: hypergrad conformal accumulation, hypergrad step with topos saturation and
//     row-wise Poincaré projection, realgrad step — fp32 as in the reference.
//
// Reference parity: AmegaHypergrad::accumulate_wave / apply (crates/st-tensor/src/pure.rs
// :10637-10815, :10585-10615), project_to_poincare (:7528-7621), porous_mix
// (crates/st-tensor/src/pure/topos.rs:169-188), AmegaRealgrad (:11315-11470),
// apply_adam_slice (crates/st-nn/src/zspace_coherence/vae.rs:303-334).
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {
using namespace st;

inline int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)st::sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
};

template <typename GradT>
__device__ __forceinline__ float load_grad(const GradT* g, long long i);
template <>
__device__ __forceinline__ float load_grad<float>(const float* g, long long i) { return g[i]; }
template <>
__device__ __forceinline__ float load_grad<__nv_bfloat16>(const __nv_bfloat16* g, long long i) {
  return __bfloat162float(g[i]);
}

template <typename GradT>
__global__ void adamw_kernel(GradT* __restrict__ grad, float* __restrict__ master,
                             float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ weight, long long n, AdamArgs a,
                             const float* __restrict__ scale_ptr, int zero_grad) {
  const float gs = a.grad_scale * (scale_ptr ? *scale_ptr : 1.0f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float g = load_grad<GradT>(grad, i) * gs;
    float w = master[i];
    float mi = a.beta1 * m[i] + (1.0f - a.beta1) * g;
    float vi = a.beta2 * v[i] + (1.0f - a.beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float mhat = mi / a.bc1;
    const float vhat = vi / a.bc2;
    w = w - a.lr * (mhat / (sqrtf(vhat) + a.eps) + a.weight_decay * w);
    master[i] = w;
    if (weight) weight[i] = __float2bfloat16(w);
    if (zero_grad) grad[i] = GradT(0.0f);
  }
}

template <typename GradT>
__global__ void sgd_kernel(GradT* __restrict__ grad, float* __restrict__ master,
                           float* __restrict__ mom, __nv_bfloat16* __restrict__ weight, long long n,
                           float lr, float momentum, float weight_decay, float grad_scale,
                           const float* __restrict__ scale_ptr, int nesterov, int zero_grad) {
  const float gs = grad_scale * (scale_ptr ? *scale_ptr : 1.0f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float w = master[i];
    float g = load_grad<GradT>(grad, i) * gs + weight_decay * w;
    if (mom) {
      const float b = momentum * mom[i] + g;
      mom[i] = b;
      g = nesterov ? g + momentum * b : b;
    }
    w -= lr * g;
    master[i] = w;
    if (weight) weight[i] = __float2bfloat16(w);
    if (zero_grad) grad[i] = GradT(0.0f);
  }
}

template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.0f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = load_grad<T>(x, i);
    s += v * v;
  }
  s = warp_sum(s);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = s;
  __syncthreads();
  if (w == 0) {
    s = l < (blockDim.x >> 5) ? sh[l] : 0.0f;
    s = warp_sum(s);
    if (l == 0) atomicAdd(out, s);
  }
}

// coef = min(1, max_norm / (sqrt(sumsq * norm_scale^2) + 1e-6)); also stores the norm.
__global__ void clip_coef_kernel(const float* sumsq, float norm_scale, float max_norm, float* coef,
                                 float* norm_out) {
  const float nrm = sqrtf(*sumsq) * norm_scale;
  if (norm_out) *norm_out = nrm;
  *coef = (max_norm > 0.0f) ? fminf(1.0f, max_norm / (nrm + 1e-6f)) : 1.0f;
}

// ---- Amegagrad ---------------------------------------------------------------------
__device__ __forceinline__ float porous_mix(float value, float saturation, float porosity) {
  if (!isfinite(value)) return 0.0f;
  if (saturation <= 0.0f) return 0.0f;
  const float limit = fabsf(saturation);
  const float mag = fabsf(value);
  if (mag <= limit) return value;
  const float sgn = value > 0.0f ? 1.0f : -1.0f;
  if (porosity <= 1.1920929e-7f) return sgn * limit;
  const float bleed = (mag - limit) / (mag + limit);
  const float absorb = fminf(porosity * 0.25f, 1.0f);
  const float softened = fmaxf(limit * (1.0f - absorb * fminf(bleed, 1.0f)), 0.0f);
  return sgn * softened;
}

// g <- sat(g + v / max(|1 - c v^2|, tol))      (conformal = 1)
// g <- sat(g + v)                               (conformal = 0: realgrad / accumulate_pair)
__global__ void hyper_accumulate_kernel(float* __restrict__ g, const float* __restrict__ v,
                                        long long n, float curvature, float tol, float saturation,
                                        float porosity, int conformal, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float x = v[i] * scale;
    float upd = x;
    if (conformal) upd = x / fmaxf(fabsf(1.0f - curvature * x * x), tol);
    g[i] = porous_mix(g[i] + upd, saturation, porosity);
  }
}

// One CTA per row: w' = sat(w - lr / max(|1 - c w^2|, tol) * g); row *= tanh(|row|/s)/|row|;
// then (optional realgrad on the projected weights) w'' = w' - lr_real * g_real; zero tapes.
__global__ void __launch_bounds__(256)
hyper_apply_kernel(float* __restrict__ w, float* __restrict__ g, float* __restrict__ g_real,
                   int rows, int cols, float curvature, float lr, float lr_real, float tol,
                   float saturation, float porosity, int use_hyper) {
  __shared__ float sh[8];
  const int row = blockIdx.x;
  float* wr = w + (size_t)row * cols;
  float ss = 0.0f;
  if (use_hyper) {
    float* gr = g + (size_t)row * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float o = wr[c];
      const float step = lr / fmaxf(fabsf(1.0f - curvature * o * o), tol);
      const float nx = porous_mix(o - step * gr[c], saturation, porosity);
      wr[c] = nx;
      gr[c] = 0.0f;
      ss += nx * nx;
    }
    ss = warp_sum(ss);
    const int wp = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) sh[wp] = ss;
    __syncthreads();
    if (wp == 0) {
      ss = l < (blockDim.x >> 5) ? sh[l] : 0.0f;
      ss = warp_sum(ss);
      if (l == 0) sh[0] = ss;
    }
    __syncthreads();
    const float norm = sqrtf(sh[0]);
    const float factor = norm > 0.0f ? tanhf(norm / sqrtf(-curvature)) / norm : 1.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float x = wr[c] * factor;
      if (g_real) {
        float* rr = g_real + (size_t)row * cols;
        x -= lr_real * rr[c];
        rr[c] = 0.0f;
      }
      wr[c] = x;
    }
  } else if (g_real) {
    float* rr = g_real + (size_t)row * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      wr[c] -= lr_real * rr[c];
      rr[c] = 0.0f;
    }
  }
}

__global__ void __launch_bounds__(256)
poincare_project_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols,
                        float curvature) {
  __shared__ float sh[8];
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * cols;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) ss += xr[c] * xr[c];
  ss = warp_sum(ss);
  const int wp = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[wp] = ss;
  __syncthreads();
  if (wp == 0) {
    ss = l < (blockDim.x >> 5) ? sh[l] : 0.0f;
    ss = warp_sum(ss);
    if (l == 0) sh[0] = ss;
  }
  __syncthreads();
  const float norm = sqrtf(sh[0]);
  const float factor = norm > 0.0f ? tanhf(norm / sqrtf(-curvature)) / norm : 1.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) y[(size_t)row * cols + c] = xr[c] * factor;
}

}  // namespace

ST_API int st_adamw(void* grad, int grad_is_bf16, float* master, float* m, float* v, void* weight,
                    long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                    int step, float grad_scale, const float* scale_ptr, int zero_grad, void* stream_v) {
  if (n <= 0) return ST_OK;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.0f - powf(beta1, (float)step);
  a.bc2 = 1.0f - powf(beta2, (float)step);
  a.grad_scale = grad_scale;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(grad), master, m, v, static_cast<__nv_bfloat16*>(weight), n, a,
        scale_ptr, zero_grad);
  else
    adamw_kernel<float><<<grid_for(n, 256), 256, 0, s>>>(
        static_cast<float*>(grad), master, m, v, static_cast<__nv_bfloat16*>(weight), n, a, scale_ptr,
        zero_grad);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_sgd(void* grad, int grad_is_bf16, float* master, float* mom, void* weight, long long n,
                  float lr, float momentum, float weight_decay, float grad_scale,
                  const float* scale_ptr, int nesterov, int zero_grad, void* stream_v) {
  if (n <= 0) return ST_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (grad_is_bf16)
    sgd_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(grad), master, mom, static_cast<__nv_bfloat16*>(weight), n, lr,
        momentum, weight_decay, grad_scale, scale_ptr, nesterov, zero_grad);
  else
    sgd_kernel<float><<<grid_for(n, 256), 256, 0, s>>>(
        static_cast<float*>(grad), master, mom, static_cast<__nv_bfloat16*>(weight), n, lr, momentum,
        weight_decay, grad_scale, scale_ptr, nesterov, zero_grad);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// out += sum(x^2).  The caller zeroes `out` before the first call of a step.
ST_API int st_sumsq(const void* x, int is_bf16, long long n, float* out, void* stream_v) {
  if (n <= 0) return ST_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (is_bf16)
    sumsq_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, out);
  else
    sumsq_kernel<float><<<grid_for(n, 256), 256, 0, s>>>(static_cast<const float*>(x), n, out);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_clip_coef(const float* sumsq, float norm_scale, float max_norm, float* coef,
                        float* norm_out, void* stream_v) {
  clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(sumsq, norm_scale, max_norm,
                                                                          coef, norm_out);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_hyper_accumulate(float* g, const float* v, long long n, float curvature, float tol,
                               float saturation, float porosity, int conformal, float scale,
                               void* stream_v) {
  if (n <= 0) return ST_OK;
  hyper_accumulate_kernel<<<grid_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      g, v, n, curvature, tol, saturation, porosity, conformal, scale);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_hyper_apply(float* w, float* g, float* g_real, int rows, int cols, float curvature,
                          float lr, float lr_real, float tol, float saturation, float porosity,
                          void* stream_v) {
  if (rows <= 0 || cols <= 0) return ST_OK;
  if (g && !(curvature < 0.0f)) return st::fail(ST_ERR_INVALID, "hypergrad: curvature must be negative");
  hyper_apply_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      w, g, g_real, rows, cols, curvature, lr, lr_real, tol, saturation, porosity, g != nullptr);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_poincare_project(const float* x, float* y, int rows, int cols, float curvature,
                               void* stream_v) {
  if (!(curvature < 0.0f)) return st::fail(ST_ERR_INVALID, "project_to_poincare: curvature must be negative");
  poincare_project_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(x, y, rows, cols, curvature);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
