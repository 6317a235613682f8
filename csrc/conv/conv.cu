// 3x3 convolution (stride 1, padding 1) as implicit GEMM on the tcgen05 kernel, plus pooling.
//
// Activations are NHWC bf16, so a block of output pixels x 64 input channels at one filter tap
// is a rectangular box of the input tensor: the TMA unit fetches it directly (zero-filling the
// halo), no im2col matrix is ever materialised.  Weights are stored [OC][tap][IC] (tap-major K).
//
//   forward        Y[p, oc]  = act(Σ_tap Σ_ic X[p + tap, ic] · W[oc, tap, ic] + bias[oc])
//   data gradient  dX[p, ic] = (Σ_tap Σ_oc dY[p + tap, oc] · Wt[ic, tap, oc]) ⊙ [X[p, ic] > 0]
//                  — the same kernel on dY with the flipped/transposed weights Wt and the ReLU mask of
//                  the layer input fused in the epilogue
//   weight gradient dW[oc, tap, ic] += Σ_p dY[p, oc] · X[p + tap, ic]
//                  — K runs over pixels, one (tap, K-split) per batch index, fp32 atomics into dW
// The first layer (3 input channels) uses a small explicit im2col (K padded to 32).
//
// Pooling: 2x2 max pool forward/backward and global average pool forward/backward on NHWC bf16.
//
// Reference parity: fused_im2col_matmul.wgsl, fused_grad_input_col2im.wgsl (crates/st-tensor/src/
// wgpu_shaders), CPU im2col path of crates/st-nn/src/layers/conv.rs:607-1017, pooling entry points
// of tensor_utils.wgsl.
#include "../gemm/gemm_kernel.cuh"
#include <cstring>

namespace {
using namespace st;
using namespace st::gemm;

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const OutMaps& tmC, const GemmParams& p,
                cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, COMM_NONE>;
  static bool configured[st::kMaxDevices] = {false};   // the attribute is per device
  const int dev = st::current_device();
  if (!configured[dev]) {
    ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured[dev] = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
  const int grid = tiles < st::sm_count() ? tiles : st::sm_count();
  GemmComm none{};
  kern<<<grid, NUM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, tmA, p, none);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// pixel block of `pixels` (128 or 64) output positions: W columns x Hb rows x Nb images
bool block_geometry(int N, int H, int W, int pixels, int* Hb, int* Nb) {
  if (W <= 0 || W > pixels || pixels % W != 0) return false;
  int hb = pixels / W;
  int nb = 1;
  if (hb > H) {
    if (hb % H != 0) return false;
    nb = hb / H;
    hb = H;
  }
  if (H % hb != 0 || N % nb != 0) return false;
  *Hb = hb;
  *Nb = nb;
  return true;
}

bool nhwc_map(CUtensorMap* out, const void* base, int N, int H, int W, int C, int Wb, int Hb, int Nb) {
  uint64_t dims[4] = {(uint64_t)C, (uint64_t)W, (uint64_t)H, (uint64_t)N};
  uint64_t strides[3] = {(uint64_t)C * 2, (uint64_t)W * C * 2, (uint64_t)H * W * C * 2};
  uint32_t box[4] = {64, (uint32_t)Wb, (uint32_t)Hb, (uint32_t)Nb};
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

__global__ void im2col3x3_small_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col,
                                       int N, int H, int W, int C, int Kpad) {
  const long long total = (long long)N * H * W * Kpad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = i % Kpad;
    const long long pix = i / Kpad;
    const int w = pix % W;
    const int h = (pix / W) % H;
    const int n = pix / ((long long)W * H);
    __nv_bfloat16 v = __float2bfloat16(0.0f);
    if (k < 9 * C) {
      const int tap = k / C, c = k - tap * C;
      const int hh = h + tap / 3 - 1, ww = w + tap % 3 - 1;
      if (hh >= 0 && hh < H && ww >= 0 && ww < W) v = x[(((long long)n * H + hh) * W + ww) * C + c];
    }
    col[i] = v;
  }
}

// Eight channels per thread (16-byte loads, one 16-byte store of y and one 8-byte store of idx); C % 8 == 0.
__global__ void __launch_bounds__(256)
maxpool2_fwd8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                     unsigned char* __restrict__ idx, int N, int H, int W, int C) {
  const int OH = H / 2, OW = W / 2, C8 = C / 8;
  const long long total = (long long)N * OH * OW * C8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c8 = i % C8;
    const long long p = i / C8;
    const int ow = p % OW;
    const int oh = (p / OW) % OH;
    const int n = p / ((long long)OW * OH);
    uint4 v[4];
#pragma unroll
    for (int t = 0; t < 4; ++t)
      v[t] = *reinterpret_cast<const uint4*>(
          x + ((((long long)n * H + oh * 2 + (t >> 1)) * W + ow * 2 + (t & 1)) * C + c8 * 8));
    float best[8];
    unsigned arg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; arg[j] = 0; }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const uint32_t w[4] = {v[t].x, v[t].y, v[t].z, v[t].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(w[q]);
        if (f.x > best[2 * q]) { best[2 * q] = f.x; arg[2 * q] = t; }
        if (f.y > best[2 * q + 1]) { best[2 * q + 1] = f.y; arg[2 * q + 1] = t; }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(best[0], best[1]); o.y = pack_bf16x2(best[2], best[3]);
    o.z = pack_bf16x2(best[4], best[5]); o.w = pack_bf16x2(best[6], best[7]);
    *reinterpret_cast<uint4*>(y + (p * C + c8 * 8)) = o;
    uint2 a;
    a.x = arg[0] | (arg[1] << 8) | (arg[2] << 16) | (arg[3] << 24);
    a.y = arg[4] | (arg[5] << 8) | (arg[6] << 16) | (arg[7] << 24);
    *reinterpret_cast<uint2*>(idx + (p * C + c8 * 8)) = a;
  }
}

// y[n, h/2, w/2, c] = max over the 2x2 window; idx (uint8) records the arg-max for the backward pass
__global__ void maxpool2_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                    unsigned char* __restrict__ idx, int N, int H, int W, int C) {
  const int OH = H / 2, OW = W / 2;
  const long long total = (long long)N * OH * OW * (C / 2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c2 = i % (C / 2);
    const long long p = i / (C / 2);
    const int ow = p % OW;
    const int oh = (p / OW) % OH;
    const int n = p / ((long long)OW * OH);
    float2 best = make_float2(-INFINITY, -INFINITY);
    int ix = 0, iy = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(
          x + ((((long long)n * H + oh * 2 + (t >> 1)) * W + ow * 2 + (t & 1)) * C + c2 * 2));
      const float2 f = __bfloat1622float2(v);
      if (f.x > best.x) { best.x = f.x; ix = t; }
      if (f.y > best.y) { best.y = f.y; iy = t; }
    }
    *reinterpret_cast<__nv_bfloat162*>(y + (p * C + c2 * 2)) = __floats2bfloat162_rn(best.x, best.y);
    idx[p * C + c2 * 2] = (unsigned char)ix;
    idx[p * C + c2 * 2 + 1] = (unsigned char)iy;
  }
}

__global__ void maxpool2_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const unsigned char* __restrict__ idx,
                                    __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C) {
  const int OH = H / 2, OW = W / 2;
  const long long total = (long long)N * OH * OW * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = i % C;
    const long long p = i / C;
    const int ow = p % OW;
    const int oh = (p / OW) % OH;
    const int n = p / ((long long)OW * OH);
    const int t = idx[i];
    const __nv_bfloat16 g = dy[i];
#pragma unroll
    for (int q = 0; q < 4; ++q)
      dx[(((long long)n * H + oh * 2 + (q >> 1)) * W + ow * 2 + (q & 1)) * C + c] =
          q == t ? g : __float2bfloat16(0.0f);
  }
}

// y[n, c] = mean over H*W
__global__ void avgpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int N,
                                   int HW, int C) {
  const int n = blockIdx.x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float s = 0.0f;
    for (int p = 0; p < HW; ++p) s += __bfloat162float(x[((long long)n * HW + p) * C + c]);
    y[(long long)n * C + c] = __float2bfloat16(s / HW);
  }
}
__global__ void avgpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, int N,
                                   int HW, int C) {
  const long long total = (long long)N * HW * C;
  const float inv = 1.0f / HW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = i % C;
    const long long n = i / ((long long)HW * C);
    dx[i] = __float2bfloat16(__bfloat162float(dy[n * C + c]) * inv);
  }
}

inline int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)st::sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

struct StConvArgs {
  const void* x;       // bf16 NHWC [N, H, W, C]
  const void* w;       // bf16 [OC, 9*C] (tap-major)
  const void* bias;    // bf16 [OC] or null
  void* y;             // bf16 NHWC [N, H, W, OC]
  const void* aux_in;  // bf16 [N*H*W, OC]: ReLU mask source for act == 4, or null
  int N, H, W, C, OC;
  int act;             // 0 none, 1 relu, 4 relu_bwd(aux_in)
};

ST_API int st_conv3x3_fwd(const StConvArgs* a, void* stream_v) {
  if (!a || !a->x || !a->w || !a->y) return st::fail(ST_ERR_INVALID, "conv3x3: null pointer");
  if (a->C % 64 != 0) return st::fail(ST_ERR_INVALID, "conv3x3: input channels must be a multiple of 64");
  if (a->OC % 8 != 0) return st::fail(ST_ERR_INVALID, "conv3x3: output channels must be a multiple of 8");
  int Hb, Nb;
  if (!block_geometry(a->N, a->H, a->W, BM, &Hb, &Nb))
    return st::fail(ST_ERR_INVALID, "conv3x3: image width must divide 128 and the batch must fill whole pixel blocks");
  const int P = a->N * a->H * a->W;
  CUtensorMap tmA, tmB;
  if (!nhwc_map(&tmA, a->x, a->N, a->H, a->W, a->C, a->W, Hb, Nb)) return ST_ERR_CUDA;
  const bool small = a->OC <= 128;
  {
    uint64_t dims[3] = {(uint64_t)9 * a->C, (uint64_t)a->OC, 1};
    uint64_t strides[2] = {(uint64_t)9 * a->C * 2, (uint64_t)9 * a->C * 2 * a->OC};
    uint32_t box[3] = {BK, (uint32_t)(small ? 128 : 256), 1};
    if (!encode_tmap(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }
  OutMaps tmC;
  memset(&tmC, 0, sizeof(tmC));
  {
    uint64_t dims[3] = {(uint64_t)a->OC, (uint64_t)P, 1};
    uint64_t strides[2] = {(uint64_t)a->OC * 2, (uint64_t)a->OC * 2 * P};
    uint32_t box[3] = {64, 32, 1};
    if (!encode_tmap(&tmC.m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->y, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }
  GemmParams p{};
  p.conv.mode = 1;
  p.conv.H = a->H; p.conv.W = a->W; p.conv.Hb = Hb; p.conv.Nb = Nb;
  p.conv.c_chunks = a->C / 64; p.conv.taps = 9;
  p.C = a->y; p.ldc = a->OC;
  p.bias = static_cast<const __nv_bfloat16*>(a->bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(a->aux_in);
  p.ld_aux_in = a->OC;
  p.M = P; p.N = a->OC; p.K = 9 * a->C;
  p.alpha = 1.0f; p.act = a->act; p.batch = 1;
  p.use_tma_store = 1;
  p.err = st::error_word();
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (small) return launch_gemm<128, 6, false, false>(tmA, tmB, tmC, p, s);
  return launch_gemm<256, 4, false, false>(tmA, tmB, tmC, p, s);
}

struct StConvWgradArgs {
  const void* dy;   // bf16 [N*H*W, OC]
  const void* x;    // bf16 NHWC [N, H, W, C]
  float* dw;        // fp32 [OC, 9*C]; the kernel ADDS into it
  int N, H, W, C, OC;
  int splits;       // K splits over pixels (0 = choose)
};

ST_API int st_conv3x3_wgrad(const StConvWgradArgs* a, void* stream_v) {
  if (!a || !a->dy || !a->x || !a->dw) return st::fail(ST_ERR_INVALID, "conv3x3_wgrad: null pointer");
  if (a->C % 64 != 0 || a->OC % 8 != 0) return st::fail(ST_ERR_INVALID, "conv3x3_wgrad: C % 64 and OC % 8 must be 0");
  int Hb, Nb;
  if (!block_geometry(a->N, a->H, a->W, BK, &Hb, &Nb))
    return st::fail(ST_ERR_INVALID, "conv3x3_wgrad: image width must divide 64 and the batch must fill whole pixel blocks");
  const int P = a->N * a->H * a->W;
  const int kblocks_total = P / BK;
  const bool small = a->C <= 128;
  const int BNv = small ? 128 : 256;
  const int tiles = ((a->OC + BM - 1) / BM) * ((a->C + BNv - 1) / BNv) * 9;
  int splits = a->splits;
  if (splits <= 0) {
    splits = (2 * st::sm_count() + tiles - 1) / tiles;
    while (splits > 1 && (kblocks_total % splits != 0 || kblocks_total / splits < 8)) --splits;
  }
  if (kblocks_total % splits != 0) return st::fail(ST_ERR_INVALID, "conv3x3_wgrad: splits must divide the pixel blocks");
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[3] = {(uint64_t)a->OC, (uint64_t)P, 1};
    uint64_t strides[2] = {(uint64_t)a->OC * 2, (uint64_t)a->OC * 2 * P};
    uint32_t box[3] = {64, BK, 1};
    if (!encode_tmap(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->dy, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }
  if (!nhwc_map(&tmB, a->x, a->N, a->H, a->W, a->C, a->W, Hb, Nb)) return ST_ERR_CUDA;
  OutMaps tmC;
  memset(&tmC, 0, sizeof(tmC));
  GemmParams p{};
  p.conv.mode = 2;
  p.conv.H = a->H; p.conv.W = a->W; p.conv.Hb = Hb; p.conv.Nb = Nb;
  p.conv.c_chunks = a->C / 64; p.conv.taps = 9;
  p.C = a->dw; p.ldc = 9ll * a->C;
  p.M = a->OC; p.N = a->C; p.K = (kblocks_total / splits) * BK;
  p.alpha = 1.0f; p.batch = 9 * splits; p.batch_stride_c = a->C;
  p.out_fp32 = 1; p.accumulate = 2;
  p.err = st::error_word();
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (small) return launch_gemm<128, 6, true, true>(tmA, tmB, tmC, p, s);
  return launch_gemm<256, 4, true, true>(tmA, tmB, tmC, p, s);
}

ST_API int st_im2col3x3_small(const void* x, void* col, int N, int H, int W, int C, int Kpad, void* stream_v) {
  if (9 * C > Kpad || (Kpad & 7)) return st::fail(ST_ERR_INVALID, "im2col: Kpad must be a multiple of 8 and >= 9*C");
  const long long total = (long long)N * H * W * Kpad;
  im2col3x3_small_kernel<<<grid_for(total, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(col), N, H, W, C, Kpad);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_maxpool2_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, void* stream_v) {
  if ((H & 1) || (W & 1) || (C & 1)) return st::fail(ST_ERR_INVALID, "maxpool2: H, W and C must be even");
  if ((C & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(idx) & 7) == 0) {
    maxpool2_fwd8_kernel<<<grid_for((long long)N * (H / 2) * (W / 2) * (C / 8), 256), 256, 0,
                           reinterpret_cast<cudaStream_t>(stream_v)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<unsigned char*>(idx), N, H, W, C);
    ST_CUDA_CHECK(cudaGetLastError());
    return ST_OK;
  }
  maxpool2_fwd_kernel<<<grid_for((long long)N * (H / 2) * (W / 2) * (C / 2), 256), 256, 0,
                        reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<unsigned char*>(idx), N, H, W, C);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
ST_API int st_maxpool2_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, void* stream_v) {
  maxpool2_bwd_kernel<<<grid_for((long long)N * (H / 2) * (W / 2) * C, 256), 256, 0,
                        reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const unsigned char*>(idx), static_cast<__nv_bfloat16*>(dx),
      N, H, W, C);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
ST_API int st_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream_v) {
  avgpool_fwd_kernel<<<N, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), N, HW, C);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
ST_API int st_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream_v) {
  avgpool_bwd_kernel<<<grid_for((long long)N * HW * C, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), N, HW, C);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
