// LayerNorm and RMSNorm, forward and backward, bf16 in / fp32 statistics.
//
// Forward: one CTA per row, 16-byte vector loads, the row stays in registers between the
// statistics pass and the normalisation pass (one HBM read, one write).
// Backward: a persistent grid; each CTA walks rows with a stride, writes dx and keeps its
// share of dgamma / dbeta in registers; per-CTA partials go to an fp32 scratch buffer that
// a second kernel reduces.  (The scratch is global memory beyond inputs and outputs.)
//
// Reference parity: layer_norm.wgsl (crates/st-tensor/src/wgpu_shaders) and the CPU
// layer_norm_affine (crates/st-tensor/src/pure.rs:3702-4058); RMSNorm is new (the
// reference has none).
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "norm.h"

namespace {
using namespace st;

constexpr int NT = 256;     // threads per CTA
constexpr int MAXV = 4;     // most 16-byte vectors per thread held in registers (d <= 8192)
// The kernels are instantiated for 1, 2 or 4 vectors per thread (d <= 2048 / 4096 / 8192): the
// per-thread arrays are sized by the template argument, so the common d = 2048 case needs a
// quarter of the registers and four times as many CTAs stay resident per SM.

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < NT / 32) ? sh[threadIdx.x] : 0.0f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) sh[0] = t;
  }
  __syncthreads();
  return sh[0];
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// RMS: y = x * rstd * gamma.   LN: y = (x - mean) * rstd * gamma + beta.
// Optional fused residual: x := x + residual is written to `sum_out` before normalising.
template <bool RMS, int MV>
__global__ void __launch_bounds__(NT)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int d,
                float eps) {
  __shared__ float sh[NT / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nvec = d >> 3;
  const __nv_bfloat16* xr = x + (size_t)row * d;
  float v[MV][8];
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int vi = threadIdx.x + i * NT;
    if (vi < nvec) {
      load8(xr + vi * 8, v[i]);
      if (residual) {
        float r[8];
        load8(residual + (size_t)row * d + vi * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        if (sum_out) {
          store8(sum_out + (size_t)row * d + vi * 8, v[i]);
          // normalise what was stored (bf16-rounded) so forward and backward agree
          load8(sum_out + (size_t)row * d + vi * 8, v[i]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += RMS ? v[i][j] * v[i][j] : v[i][j];
    }
  }
  float mean = 0.0f, rstd;
  if (RMS) {
    const float ms = block_sum(s, sh) / d;
    rstd = rsqrtf(ms + eps);
  } else {
    mean = block_sum(s, sh) / d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float c = v[i][j] - mean;
          q += c * c;
        }
      }
    }
    const float var = block_sum(q, sh) / d;
    rstd = rsqrtf(var + eps);
  }
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int vi = threadIdx.x + i * NT;
    if (vi < nvec) {
      float g[8], o[8];
      load8(gamma + vi * 8, g);
      if (!RMS && beta) {
        float b[8];
        load8(beta + vi * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + b[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j];
      }
      store8(y + (size_t)row * d + vi * 8, o);
    }
  }
}

// dx for one row and the CTA's running dgamma/dbeta.
template <bool RMS, int MV>
__global__ void __launch_bounds__(NT)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial_dgamma,
                float* __restrict__ partial_dbeta, int rows, int d) {
  __shared__ float sh[NT / 32];
  const int nvec = d >> 3;
  float g[MV][8], dg[MV][8], db[MV][8];
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int vi = threadIdx.x + i * NT;
    if (vi < nvec) load8(gamma + vi * 8, g[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[i][j] = 0.0f;
      db[i][j] = 0.0f;
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mean = RMS ? 0.0f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[MV][8], gy[MV][8], rr[MV][8];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
        float xv[8], dv[8];
        load8(x + (size_t)row * d + vi * 8, xv);
        load8(dy + (size_t)row * d + vi * 8, dv);
        // the residual-branch gradient is only needed after the row reduction: issue its load now so that the
        // reduction hides the latency
        if (dres) load8(dres + (size_t)row * d + vi * 8, rr[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          gy[i][j] = dv[j] * g[i][j];
          dg[i][j] += dv[j] * xh[i][j];
          db[i][j] += dv[j];
          s1 += gy[i][j] * xh[i][j];
          s2 += gy[i][j];
        }
      }
    }
    const float m1 = block_sum(s1, sh) / d;
    const float m2 = RMS ? 0.0f : block_sum(s2, sh) / d;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gy[i][j] - m2 - xh[i][j] * m1);
        if (dres) {  // gradient arriving through the residual branch
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rr[i][j];
        }
        store8(dx + (size_t)row * d + vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int vi = threadIdx.x + i * NT;
    if (vi < nvec) {
      float* pg = partial_dgamma + (size_t)blockIdx.x * d + vi * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) pg[j] = dg[i][j];
      if (!RMS && partial_dbeta) {
        float* pb = partial_dbeta + (size_t)blockIdx.x * d + vi * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) pb[j] = db[i][j];
      }
    }
  }
}

// out[c] (+)= sum_p partial[p, c].  A CTA owns 32 columns; its 8 thread rows sum every 8th partial
// (each a coalesced 128-byte read) and are combined through shared memory.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts, int d, int accumulate) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, k = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s0 = 0.0f, s1 = 0.0f;
  if (c < d) {
    int p = k;
    for (; p + 8 < parts; p += 16) {
      s0 += partial[(size_t)p * d + c];
      s1 += partial[(size_t)(p + 8) * d + c];
    }
    if (p < parts) s0 += partial[(size_t)p * d + c];
  }
  sh[k][cx] = s0 + s1;
  __syncthreads();
  if (k == 0 && c < d) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sh[i][cx];
    out[c] = accumulate ? out[c] + t : t;
  }
}

}  // namespace

namespace st {
int norm_bwd_grid(int rows) {
  int g = sm_count() * 2;
  return rows < g ? rows : g;
}
// CTAs for the regular entry: as many as stay resident (register footprint grows with d)
int norm_bwd_grid_for(int rows, int d) {
  const int per_sm = d <= 2048 ? 4 : 2;
  int g = sm_count() * per_sm;
  return rows < g ? rows : g;
}
}  // namespace st

static int check_dims(int rows, int d) {
  if (rows <= 0 || d <= 0) return st::fail(ST_ERR_INVALID, "norm: non-positive dimension");
  if (d & 7) return st::fail(ST_ERR_INVALID, "norm: feature dimension must be a multiple of 8");
  if (d > NT * MAXV * 8) return st::fail(ST_ERR_TOO_LARGE, "norm: feature dimension above 8192");
  return ST_OK;
}

ST_API int st_norm_fwd(int rms, const void* x, const void* residual, const void* gamma,
                       const void* beta, void* y, void* sum_out, float* mean, float* rstd, int rows,
                       int d, float eps, void* stream_v) {
  if (int e = check_dims(rows, d)) return e;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto B = static_cast<const __nv_bfloat16*>(beta);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto S = static_cast<__nv_bfloat16*>(sum_out);
#define ST_NORM_FWD(RMSV, MVV) norm_fwd_kernel<RMSV, MVV><<<rows, NT, 0, s>>>(X, R, G, B, Y, S, mean, rstd, rows, d, eps)
  const int mv = d <= NT * 8 ? 1 : (d <= NT * 16 ? 2 : 4);
  if (rms) {
    if (mv == 1) ST_NORM_FWD(true, 1); else if (mv == 2) ST_NORM_FWD(true, 2); else ST_NORM_FWD(true, 4);
  } else {
    if (mv == 1) ST_NORM_FWD(false, 1); else if (mv == 2) ST_NORM_FWD(false, 2); else ST_NORM_FWD(false, 4);
  }
#undef ST_NORM_FWD
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// Number of fp32 scratch elements st_norm_bwd needs for `rows` x `d`.
ST_API long long st_norm_bwd_scratch_elems(int rows, int d) {
  return 2ll * st::norm_bwd_grid_for(rows, d) * d;
}

int st::norm_bwd_launch(int rms, const void* dy, const void* x, const void* gamma,
                        const float* mean, const float* rstd, const void* dres, void* dx,
                        float* dgamma, float* dbeta, int accumulate, float* scratch, int rows,
                        int d, int grid, cudaStream_t s) {
  if (int e = check_dims(rows, d)) return e;
  if (grid < 1) return st::fail(ST_ERR_INVALID, "norm_bwd: grid must be positive");
  float* pg = scratch;
  float* pb = scratch + (size_t)grid * d;
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
#define ST_NORM_BWD(RMSV, MVV, PB) norm_bwd_kernel<RMSV, MVV><<<grid, NT, 0, s>>>(DY, X, G, mean, rstd, DR, DX, pg, PB, rows, d)
  const int mv = d <= NT * 8 ? 1 : (d <= NT * 16 ? 2 : 4);
  if (rms) {
    if (mv == 1) ST_NORM_BWD(true, 1, nullptr); else if (mv == 2) ST_NORM_BWD(true, 2, nullptr); else ST_NORM_BWD(true, 4, nullptr);
  } else {
    if (mv == 1) ST_NORM_BWD(false, 1, pb); else if (mv == 2) ST_NORM_BWD(false, 2, pb); else ST_NORM_BWD(false, 4, pb);
  }
#undef ST_NORM_BWD
  ST_CUDA_CHECK(cudaGetLastError());
  reduce_partials_kernel<<<(d + 31) / 32, 256, 0, s>>>(pg, dgamma, grid, d, accumulate);
  if (!rms && dbeta)
    reduce_partials_kernel<<<(d + 31) / 32, 256, 0, s>>>(pb, dbeta, grid, d, accumulate);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// dgamma / dbeta are fp32 [d]; with accumulate != 0 the kernel adds to them.
ST_API int st_norm_bwd(int rms, const void* dy, const void* x, const void* gamma,
                       const float* mean, const float* rstd, const void* dres, void* dx,
                       float* dgamma, float* dbeta, int accumulate, float* scratch, int rows,
                       int d, void* stream_v) {
  if (!scratch) return st::fail(ST_ERR_INVALID, "norm_bwd: scratch buffer is required");
  return st::norm_bwd_launch(rms, dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, accumulate,
                             scratch, rows, d, st::norm_bwd_grid_for(rows, d), reinterpret_cast<cudaStream_t>(stream_v));
}

// ------------------------------------------------------------------------------------------
// Entry point that allocates nothing (see norm_noalloc.h).
// ------------------------------------------------------------------------------------------
#include "norm_noalloc.h"
#include <cstdio>

// Scratch for the per-CTA dgamma / dbeta partials.  In host code this name is only a handle
// for cudaGetSymbolAddress; the kernels get the real device address as an argument.
static __device__ __align__(256) float g_norm_bwd_static_scratch[ST_NORM_BWD_NOALLOC_MAX_ELEMS];

namespace {
constexpr int kNoallocMaxDevices = 16;
float* g_noalloc_ptr[kNoallocMaxDevices] = {nullptr};
}  // namespace

ST_API int st_norm_bwd_noalloc(int rms, const void* dy, const void* x, const void* gamma,
                               const float* mean, const float* rstd, const void* dres, void* dx,
                               float* dgamma, float* dbeta, int accumulate, int rows, int d,
                               void* stream_v) {
  if (rows <= 0 || d <= 0) return st::fail(ST_ERR_INVALID, "norm_bwd_noalloc: non-positive dimension");
  const long long need = 2ll * st::norm_bwd_grid(rows) * d;
  if (need > (long long)ST_NORM_BWD_NOALLOC_MAX_ELEMS) {
    char buf[200];
    snprintf(buf, sizeof(buf),
             "norm_bwd_noalloc: rows=%d d=%d needs %lld scratch floats, the built-in buffer holds %d; "
             "use st_norm_bwd with a caller-provided scratch buffer",
             rows, d, need, (int)ST_NORM_BWD_NOALLOC_MAX_ELEMS);
    return st::fail(ST_ERR_TOO_LARGE, buf);
  }
  int dev = 0;
  ST_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoallocMaxDevices) return st::fail(ST_ERR_INVALID, "norm_bwd_noalloc: device index out of range");
  if (g_noalloc_ptr[dev] == nullptr) {
    // once per device, with that device current: resolve the array's device address
    float* p = nullptr;
    ST_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_bwd_static_scratch));
    if (p == nullptr) return st::fail(ST_ERR_CUDA, "norm_bwd_noalloc: cudaGetSymbolAddress returned null");
    g_noalloc_ptr[dev] = p;
  }
  return st::norm_bwd_launch(rms, dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, accumulate,
                             g_noalloc_ptr[dev], rows, d, st::norm_bwd_grid(rows), reinterpret_cast<cudaStream_t>(stream_v));
}
