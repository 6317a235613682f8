// Bandwidth-bound kernels of the transformer / classifier paths: RoPE, GELU forward and
// backward (+ bias-gradient column sums), column sums, embedding gather / scatter-add,
// row softmax (+ hardmax mask), cross-entropy statistics and gradient (vocab-shard aware).
//
// Reference parity: tensor_utils.wgsl entry points (embedding_gather, embedding_scatter_add,
// categorical_cross_entropy_*, relu, sum_axis0 ...), fused_gelu_back.wgsl + reduce_db.wgsl,
// softmax_*.wgsl / row_softmax_hardmax (crates/st-tensor/src/pure.rs:3277,11921).
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {
using namespace st;

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

// ------------------------------------------------------------------------------------
// RoPE (rotate-half convention), in place on `heads` consecutive heads of each row.
// x: [T, ld]; head h of row t starts at x + t*ld + h*D.  cos/sin: [S, D/2] fp32.
// ------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs,
                            const float* __restrict__ sn, long long T, int heads, int D,
                            long long ld, int seq_len, int pos_offset, float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;
  const long long total = T * heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = i % vec_per_head;
    const long long th = i / vec_per_head;
    const int h = th % heads;
    const long long t = th / heads;
    const int pos = (int)(t % seq_len) + pos_offset;
    __nv_bfloat16* p = x + t * ld + (long long)h * D + v * 8;
    float a[8], b[8], c[8], s[8];
    load8(p, a);
    load8(p + half, b);
    const float4* cp = reinterpret_cast<const float4*>(cs + (long long)pos * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sn + (long long)pos * half + v * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
    float oa[8], ob[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = sign * s[j];
      oa[j] = a[j] * c[j] - b[j] * sj;
      ob[j] = b[j] * c[j] + a[j] * sj;
    }
    store8(p, oa);
    store8(p + half, ob);
  }
}

// ------------------------------------------------------------------------------------
// GELU(tanh) forward / backward, ReLU backward; optional bias-gradient column sums.
// ------------------------------------------------------------------------------------
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                long long n8, int relu) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = relu ? fmaxf(v[j], 0.0f) : gelu_tanh(v[j]);
    store8(y + i * 8, v);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, long long n8, int relu) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8], g[8];
    load8(x + i * 8, v);
    load8(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= relu ? (v[j] > 0.0f ? 1.0f : 0.0f) : gelu_tanh_grad(v[j]);
    store8(dx + i * 8, g);
  }
}

// out[c] (+)= sum_r x[r, c]; grid (ceil(cols/32), row_chunks); fp32 atomics across chunks.
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                              long long rows, int cols, long long ld) {
  __shared__ float sh[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const long long rows_per = (rows + gridDim.y - 1) / gridDim.y;
  const long long r0 = blockIdx.y * rows_per;
  const long long r1 = min(rows, r0 + rows_per);
  float s = 0.0f;
  if (c < cols)
    for (long long r = r0 + threadIdx.y; r < r1; r += 32) s += __bfloat162float(x[r * ld + c]);
  sh[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  float t = sh[threadIdx.x][threadIdx.y];
  t = warp_sum(t);
  const int cc = blockIdx.x * 32 + threadIdx.y;
  if (threadIdx.x == 0 && cc < cols) atomicAdd(out + cc, t);
}

// Vectorised variant: each thread owns 8 adjacent columns (one 16-byte load per row) and block.y = 8
// row lanes; four rows are in flight per thread.  Needs cols % 8 == 0 and 16-byte aligned rows.
__global__ void __launch_bounds__(256)
colsum8_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long rows, int cols, long long ld) {
  __shared__ float sh[8][32 * 8 + 1];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const long long rows_per = (rows + gridDim.y - 1) / gridDim.y;
  const long long r0 = blockIdx.y * rows_per;
  const long long r1 = min(rows, r0 + rows_per);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  if (c0 < cols) {
    long long r = r0 + threadIdx.y;
    for (; r + 24 < r1; r += 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(x + (r + 8 * u) * ld + c0);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16x2(w[q]);
          acc[2 * q] += f.x;
          acc[2 * q + 1] += f.y;
        }
      }
    }
    for (; r < r1; r += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + c0);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(w[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[threadIdx.y][threadIdx.x * 8 + j] = acc[j];
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;   // 256 threads, one column each
  float s = 0.0f;
#pragma unroll
  for (int y = 0; y < 8; ++y) s += sh[y][t];
  const int c = blockIdx.x * 256 + t;
  if (c < cols) atomicAdd(out + c, s);
}

// ------------------------------------------------------------------------------------
// Embedding
// ------------------------------------------------------------------------------------
// out[t, :] = W[idx[t] - vocab_start, :] (zero when the id is outside this shard) (+ pos[t % S, :])
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ W,
                                     const __nv_bfloat16* __restrict__ pos, __nv_bfloat16* __restrict__ out,
                                     long long T, int d, int vocab_start, int vocab_local, int seq_len) {
  const int vec = d >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < T * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int v = i % vec;
    const long long id = idx[t] - vocab_start;
    float e[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (id >= 0 && id < vocab_local) load8(W + id * d + v * 8, e);
    if (pos) {
      float p[8];
      load8(pos + (t % seq_len) * d + v * 8, p);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] += p[j];
    }
    store8(out + t * d + v * 8, e);
  }
}
// dW[idx[t] - vocab_start, :] += dy[t, :]   (fp32 accumulation)
// Four fp32 additions to 16-byte aligned global memory in one reduction instruction.
__device__ __forceinline__ void red_add4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ dW, float* __restrict__ dpos, long long T, int d,
                                     int vocab_start, int vocab_local, int seq_len, int vec4) {
  // vec4: both tables start on a 16-byte boundary, so the additions can go out four at a time
  const int vec = d >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < T * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int v = i % vec;
    const long long id = idx[t] - vocab_start;
    float g[8];
    load8(dy + t * d + v * 8, g);
    if (id >= 0 && id < vocab_local) {
      float* w = dW + id * d + v * 8;
      if (vec4) {
        red_add4(w, g[0], g[1], g[2], g[3]);
        red_add4(w + 4, g[4], g[5], g[6], g[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(w + j, g[j]);
      }
    }
    if (dpos) {
      float* w = dpos + (t % seq_len) * d + v * 8;
      if (vec4) {
        red_add4(w, g[0], g[1], g[2], g[3]);
        red_add4(w + 4, g[4], g[5], g[6], g[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(w + j, g[j]);
      }
    }
  }
}

// Deterministic variant: the token positions have been sorted by id (stably) on the host side, so one CTA owns
// one distinct id and adds its occurrences in position order into registers; nothing is added atomically and
// the result does not depend on scheduling.
__global__ void embedding_bwd_sorted_kernel(const long long* __restrict__ uniq_ids, const long long* __restrict__ seg_start,
                                            const long long* __restrict__ seg_count, const long long* __restrict__ perm,
                                            const __nv_bfloat16* __restrict__ dy, float* __restrict__ dW, int d,
                                            int vocab_start, int vocab_local) {
  const long long id = uniq_ids[blockIdx.x] - vocab_start;
  if (id < 0 || id >= vocab_local) return;
  const long long start = seg_start[blockIdx.x], count = seg_count[blockIdx.x];
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long j = 0; j < count; ++j) {
      float g[8];
      load8(dy + perm[start + j] * d + c, g);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += g[k];
    }
    float* w = dW + id * d + c;
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] += acc[k];
  }
}

// ------------------------------------------------------------------------------------
// Row softmax (fp32 in/out, any width) with optional hardmax mask — Tensor API parity.
// ------------------------------------------------------------------------------------
__global__ void row_softmax_kernel(const float* __restrict__ x, float* __restrict__ y,
                                   float* __restrict__ hard, int rows, int cols) {
  __shared__ float sh[32];
  __shared__ int shi[32];
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * cols;
  float m = -INFINITY;
  int mi = 0x7fffffff;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = xr[c];
    if (v > m || (v == m && c < mi)) { m = v; mi = c; }
  }
  // block arg-max, lowest index wins ties
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
    if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) { sh[w] = m; shi[w] = mi; }
  __syncthreads();
  if (w == 0) {
    m = l < nw ? sh[l] : -INFINITY;
    mi = l < nw ? shi[l] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    if (l == 0) { sh[0] = m; shi[0] = mi; }
  }
  __syncthreads();
  m = sh[0];
  mi = shi[0];
  __syncthreads();
  float s = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(xr[c] - m);
  s = warp_sum(s);
  if (l == 0) sh[w] = s;
  __syncthreads();
  if (w == 0) {
    s = l < nw ? sh[l] : 0.0f;
    s = warp_sum(s);
    if (l == 0) sh[0] = s;
  }
  __syncthreads();
  const float inv = 1.0f / sh[0];
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    y[(size_t)row * cols + c] = __expf(xr[c] - m) * inv;
    if (hard) hard[(size_t)row * cols + c] = (c == mi) ? 1.0f : 0.0f;
  }
}

// Row softmax + arg-max mask + "spiral consensus" blend and the Z-space projection of the row, in one pass over
// the row (the reference runs three shaders: softmax, softmax_spiral_consensus.wgsl, softmax_zspace_projection.wgsl):
//   spiral[c]  = (1 + enrichment) * (phi_conj * p[c] + phi_bias * mask[c]),
//                enrichment = leech_scale * (entropy * ramanujan_ratio + hardmass * phi)
//   metrics    = (entropy, hardmass, enrichment, coherence)           per row
//   zmetrics   = (focus = sum p^2, above, here, swirl = sum p sin(c * golden_angle))  with golden-ratio bands
struct SpiralConsts {
  float phi, phi_conj, phi_bias, leech_scale, ramanujan_ratio, golden_angle;
};

__global__ void row_softmax_spiral_kernel(const float* __restrict__ x, float* __restrict__ y, float* __restrict__ hard,
                                          float* __restrict__ spiral, float* __restrict__ metrics,
                                          float* __restrict__ zmetrics, int rows, int cols, SpiralConsts k) {
  __shared__ float sh[32];
  __shared__ int shi[32];
  __shared__ float red[5][32];
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * cols;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  float m = -INFINITY;
  int mi = 0x7fffffff;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = xr[c];
    if (v > m || (v == m && c < mi)) { m = v; mi = c; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
    if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
  }
  if (l == 0) { sh[w] = m; shi[w] = mi; }
  __syncthreads();
  if (w == 0) {
    m = l < nw ? sh[l] : -INFINITY;
    mi = l < nw ? shi[l] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    if (l == 0) { sh[0] = m; shi[0] = mi; }
  }
  __syncthreads();
  m = sh[0];
  mi = shi[0];
  __syncthreads();
  float s = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(xr[c] - m);
  s = warp_sum(s);
  if (l == 0) sh[w] = s;
  __syncthreads();
  if (w == 0) {
    s = l < nw ? sh[l] : 0.0f;
    s = warp_sum(s);
    if (l == 0) sh[0] = s;
  }
  __syncthreads();
  const float inv = 1.0f / sh[0];
  // golden-ratio bands of the Z-space projection
  int band_above = max(1, (int)floorf((float)cols / k.phi));
  int band_here = max(1, (int)floorf((float)cols / (k.phi * k.phi)));
  if (band_above >= cols) { band_above = cols; band_here = 0; }
  else if (band_above + band_here >= cols) band_here = cols - band_above;
  const int band_split = band_above + band_here;
  float acc[5] = {0, 0, 0, 0, 0};   // entropy, focus, above, here, swirl
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float p = __expf(xr[c] - m) * inv;
    y[(size_t)row * cols + c] = p;
    if (hard) hard[(size_t)row * cols + c] = (c == mi) ? 1.0f : 0.0f;
    if (p > 0.0f) acc[0] -= p * __logf(p);
    acc[1] += p * p;
    if (c < band_above) acc[2] += p;
    else if (c < band_split) acc[3] += p;
    acc[4] += p * __sinf((float)c * k.golden_angle);
  }
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    const float v = warp_sum(acc[i]);
    if (l == 0) red[i][w] = v;
  }
  __syncthreads();
  if (w == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) {
      float v = l < nw ? red[i][l] : 0.0f;
      v = warp_sum(v);
      if (l == 0) red[i][0] = v;
    }
  }
  __syncthreads();
  const float entropy = red[0][0], hardmass = 1.0f;
  const float geodesic = entropy * k.ramanujan_ratio + hardmass * k.phi;
  const float enrichment = geodesic > 1e-12f ? k.leech_scale * geodesic : 0.0f;
  const float scale = 1.0f + enrichment;
  if (spiral) {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float p = y[(size_t)row * cols + c];
      spiral[(size_t)row * cols + c] = scale * (k.phi_conj * p + ((c == mi) ? k.phi_bias : 0.0f));
    }
  }
  if (threadIdx.x == 0) {
    if (metrics) {
      const float en = entropy > 0.0f ? fminf(1.0f, entropy / (entropy + 1.0f)) : 0.0f;
      const float hn = fminf(1.0f, hardmass / (float)cols);
      const float rn = enrichment != 0.0f ? fminf(1.0f, fmaxf(0.0f, enrichment / (1.0f + fabsf(enrichment)))) : 0.0f;
      float* mr = metrics + (size_t)row * 4;
      mr[0] = entropy; mr[1] = hardmass; mr[2] = enrichment; mr[3] = (en + hn + rn) / 3.0f;
    }
    if (zmetrics) {
      float* zr = zmetrics + (size_t)row * 4;
      zr[0] = red[1][0]; zr[1] = red[2][0]; zr[2] = red[3][0]; zr[3] = red[4][0];   // the row sums to one: no rescale
    }
  }
}

// ------------------------------------------------------------------------------------
// Cross-entropy over (a shard of) the vocabulary.
// stats pass: per row max, sum exp(l - max), target logit (0 when the target is elsewhere).
// grad pass : dlogits = (exp(l - lse) - [col == target]) * coef[row-independent scalar]
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                float* __restrict__ row_max, float* __restrict__ row_sum, float* __restrict__ tgt_logit,
                long long ld, int V, int vocab_start) {
  __shared__ float shm[16], shs[16];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  float m = -INFINITY, s = 0.0f;
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    load8(lr + v * 8, f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int c = (nvec << 3) + threadIdx.x; c < V; c += blockDim.x) {
    const float f = __bfloat162float(lr[c]);
    if (f > m) {
      s *= __expf(m - f);
      m = f;
    }
    s += __expf(f - m);
  }
  // combine (m, s) pairs
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.0f : s * __expf(m - nm)) + (om == -INFINITY ? 0.0f : os * __expf(om - nm));
    m = nm;
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) { shm[w] = m; shs[w] = s; }
  __syncthreads();
  if (w == 0) {
    m = l < nw ? shm[l] : -INFINITY;
    s = l < nw ? shs[l] : 0.0f;
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.0f : s * __expf(m - nm)) + (om == -INFINITY ? 0.0f : os * __expf(om - nm));
      m = nm;
    }
    if (l == 0) {
      row_max[row] = m;
      row_sum[row] = s;
      const long long t = target[row] - vocab_start;
      tgt_logit[row] = (t >= 0 && t < V) ? __bfloat162float(lr[t]) : 0.0f;
    }
  }
}

__global__ void __launch_bounds__(512)
ce_grad_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
               const float* __restrict__ lse, const float* __restrict__ coef_ptr, float coef,
               __nv_bfloat16* __restrict__ dlogits, long long ld, int V, int vocab_start,
               long long ignore_index) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  __nv_bfloat16* dr = dlogits + row * ld;
  const long long tg = target[row];
  const float k = (tg == ignore_index) ? 0.0f : coef * (coef_ptr ? *coef_ptr : 1.0f);
  const long long t = tg - vocab_start;
  const float L = lse[row];
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    load8(lr + v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(f[j] - L);
      f[j] = (p - ((long long)(v * 8 + j) == t ? 1.0f : 0.0f)) * k;
    }
    store8(dr + v * 8, f);
  }
  for (int c = (nvec << 3) + threadIdx.x; c < V; c += blockDim.x) {
    const float p = __expf(__bfloat162float(lr[c]) - L);
    dr[c] = __float2bfloat16((p - ((long long)c == t ? 1.0f : 0.0f)) * k);
  }
}

inline int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)st::sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

ST_API int st_rope(void* x, const float* cos_t, const float* sin_t, long long T, int heads, int D,
                   long long ld, int seq_len, int pos_offset, int backward, void* stream_v) {
  if (D % 16 != 0 || (ld & 7) || (reinterpret_cast<uintptr_t>(x) & 15))
    return st::fail(ST_ERR_INVALID, "rope: head_dim must be a multiple of 16 and rows 16-byte aligned");
  const long long total = T * heads * (D / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<__nv_bfloat16*>(x), cos_t, sin_t, T, heads, D, ld, seq_len, pos_offset,
      backward ? -1.0f : 1.0f);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_act_fwd(const void* x, void* y, long long n, int relu, void* stream_v) {
  if (n & 7) return st::fail(ST_ERR_INVALID, "act: element count must be a multiple of 8");
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n / 8, relu);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
ST_API int st_act_bwd(const void* x, const void* dy, void* dx, long long n, int relu, void* stream_v) {
  if (n & 7) return st::fail(ST_ERR_INVALID, "act: element count must be a multiple of 8");
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(dx), n / 8, relu);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// out (fp32 [cols]) += column sums of x (bf16 [rows, cols], leading dimension ld).
// The caller zeroes `out` first unless it wants accumulation.
ST_API int st_colsum(const void* x, float* out, long long rows, int cols, long long ld, void* stream_v) {
  if ((cols & 7) == 0 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    int chunks = (int)((rows + 255) / 256);
    if (chunks < 1) chunks = 1;
    if (chunks > 512) chunks = 512;
    colsum8_kernel<<<dim3((cols + 255) / 256, chunks), dim3(32, 8), 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
        static_cast<const __nv_bfloat16*>(x), out, rows, cols, ld);
    ST_CUDA_CHECK(cudaGetLastError());
    return ST_OK;
  }
  dim3 block(32, 32);
  int chunks = (int)((rows + 1023) / 1024);
  if (chunks < 1) chunks = 1;
  if (chunks > 256) chunks = 256;
  dim3 grid((cols + 31) / 32, chunks);
  colsum_kernel<<<grid, block, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(x), out, rows, cols, ld);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_embedding_fwd(const long long* idx, const void* W, const void* pos, void* out,
                            long long T, int d, int vocab_start, int vocab_local, int seq_len,
                            void* stream_v) {
  if (d & 7) return st::fail(ST_ERR_INVALID, "embedding: dim must be a multiple of 8");
  embedding_fwd_kernel<<<grid_for(T * (d / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      idx, static_cast<const __nv_bfloat16*>(W), static_cast<const __nv_bfloat16*>(pos),
      static_cast<__nv_bfloat16*>(out), T, d, vocab_start, vocab_local, seq_len > 0 ? seq_len : 1);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
ST_API int st_embedding_bwd(const long long* idx, const void* dy, float* dW, float* dpos, long long T,
                            int d, int vocab_start, int vocab_local, int seq_len, void* stream_v) {
  if (d & 7) return st::fail(ST_ERR_INVALID, "embedding: dim must be a multiple of 8");
  embedding_bwd_kernel<<<grid_for(T * (d / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      idx, static_cast<const __nv_bfloat16*>(dy), dW, dpos, T, d, vocab_start, vocab_local,
      seq_len > 0 ? seq_len : 1,
      ((reinterpret_cast<uintptr_t>(dW) | reinterpret_cast<uintptr_t>(dpos)) & 15) == 0 ? 1 : 0);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// Scatter-add with a fixed summation order: `uniq_ids` / `seg_start` / `seg_count` describe the runs of equal ids in
// the stably sorted id list and `perm` maps sorted positions back to rows of dy.
ST_API int st_embedding_bwd_sorted(const long long* uniq_ids, const long long* seg_start, const long long* seg_count,
                                   const long long* perm, const void* dy, float* dW, long long n_unique, int d,
                                   int vocab_start, int vocab_local, void* stream_v) {
  if (d & 7) return st::fail(ST_ERR_INVALID, "embedding: dim must be a multiple of 8");
  if (n_unique <= 0) return ST_OK;
  const int threads = d >= 2048 ? 256 : (d >= 512 ? 64 : 32);
  embedding_bwd_sorted_kernel<<<(unsigned)n_unique, threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      uniq_ids, seg_start, seg_count, perm, static_cast<const __nv_bfloat16*>(dy), dW, d, vocab_start, vocab_local);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_row_softmax_f32(const float* x, float* y, float* hard, int rows, int cols, void* stream_v) {
  if (rows <= 0 || cols <= 0) return st::fail(ST_ERR_INVALID, "softmax: empty input");
  int threads = cols >= 1024 ? 256 : (cols >= 128 ? 128 : 32);
  row_softmax_kernel<<<rows, threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(x, y, hard, rows, cols);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_row_softmax_spiral_f32(const float* x, float* y, float* hard, float* spiral, float* metrics,
                                     float* zmetrics, int rows, int cols, float phi, float phi_conj, float phi_bias,
                                     float leech_scale, float ramanujan_ratio, float golden_angle, void* stream_v) {
  if (rows <= 0 || cols <= 0) return st::fail(ST_ERR_INVALID, "softmax: empty input");
  if (!x || !y) return st::fail(ST_ERR_INVALID, "softmax: null pointer");
  int threads = cols >= 1024 ? 256 : (cols >= 128 ? 128 : 32);
  SpiralConsts k{phi, phi_conj, phi_bias, leech_scale, ramanujan_ratio, golden_angle};
  row_softmax_spiral_kernel<<<rows, threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(x, y, hard, spiral, metrics,
                                                                                           zmetrics, rows, cols, k);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_ce_stats(const void* logits, const long long* target, float* row_max, float* row_sum,
                       float* tgt_logit, long long rows, long long ld, int V, int vocab_start,
                       void* stream_v) {
  if ((ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15))
    return st::fail(ST_ERR_INVALID, "ce: logits rows must be 16-byte aligned");
  const int threads = V >= 8192 ? 512 : 128;
  ce_stats_kernel<<<(unsigned)rows, threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(logits), target, row_max, row_sum, tgt_logit, ld, V, vocab_start);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
ST_API int st_ce_grad(const void* logits, const long long* target, const float* lse,
                      const float* coef_ptr, float coef, void* dlogits, long long rows, long long ld,
                      int V, int vocab_start, long long ignore_index, void* stream_v) {
  if ((ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(dlogits) & 15))
    return st::fail(ST_ERR_INVALID, "ce: logits rows must be 16-byte aligned");
  const int threads = V >= 8192 ? 512 : 128;
  ce_grad_kernel<<<(unsigned)rows, threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(logits), target, lse, coef_ptr, coef,
      static_cast<__nv_bfloat16*>(dlogits), ld, V, vocab_start, ignore_index);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// ---- N-d indexer: logical element id -> strided address and segment id ------------------------------------------------
// Each logical id is decoded against `dims` (innermost last; a zero dimension is skipped and leaves coordinate 0),
// dotted with `strides`, and the address is bucketed into `segments` segments of `segment_stride` elements.
namespace {
struct NdIndexerParams {
  unsigned dims[4];
  unsigned strides[4];
  unsigned segments, segment_stride;
};

__global__ void nd_indexer_kernel(const unsigned* __restrict__ positions, unsigned* __restrict__ out_index,
                                  unsigned* __restrict__ out_segment, long long n, NdIndexerParams p) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    unsigned remaining = positions[i], flat = 0;
#pragma unroll
    for (int d = 3; d >= 0; --d) {
      const unsigned dim = p.dims[d];
      if (dim == 0) continue;
      flat += (remaining % dim) * p.strides[d];
      remaining /= dim;
    }
    out_index[i] = flat;
    out_segment[i] = (flat / p.segment_stride) % p.segments;
  }
}
}  // namespace

ST_API int st_nd_indexer(const unsigned* positions, unsigned* out_index, unsigned* out_segment, long long n,
                         const unsigned* dims4, const unsigned* strides4, unsigned segments, unsigned segment_stride,
                         void* stream_v) {
  if (n <= 0) return ST_OK;
  if (!dims4 || !strides4) return st::fail(ST_ERR_INVALID, "nd_indexer: null dims / strides");
  if (segments == 0 || segment_stride == 0) return st::fail(ST_ERR_INVALID, "nd_indexer: segments and segment_stride must be positive");
  NdIndexerParams p;
  for (int i = 0; i < 4; ++i) { p.dims[i] = dims4[i]; p.strides[i] = strides4[i]; }
  p.segments = segments; p.segment_stride = segment_stride;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  nd_indexer_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(positions, out_index, out_segment, n, p);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
