// Persistent bf16 GEMM for sm_100a: C[M,N] = epilogue(alpha * A·Bᵀ).
//
//   * operands arrive by TMA (128-byte swizzle) into a 4-stage shared-memory ring;
//   * one elected thread issues tcgen05.mma (128 x BN x 16, cta_group::1) with fp32
//     accumulators in TMEM; two accumulator buffers let the epilogue of tile i overlap the
//     main loop of tile i+1;
//   * four epilogue warps read TMEM with tcgen05.ld and apply the fused epilogue:
//     +bias, ReLU / GELU(tanh), store of the pre-activation, multiply by GELU'/ReLU' of a
//     saved pre-activation (backward), +residual, C += (gradient accumulation), bf16 or
//     fp32 output.
//
// Operand layouts.  "K-major" A is a row-major [M,K] matrix, "MN-major" A is a row-major
// [K,M] matrix (i.e. Aᵀ is what is stored).  Same for B with N in place of M.  This covers
// forward (K,K), data-gradient (K,MN) and weight-gradient (MN,MN) products of a linear
// layer without any transposition pass.
//
// Parity with the reference: replaces dense_matmul.wgsl / fused_matmul_bias_*.wgsl
// (crates/st-tensor/src/wgpu_shaders) and rocBLAS sgemm + hip_gemm_epilogue.cu
// (crates/st-backend-hip/src/real.rs:759-960).
#include "gemm_kernel.cuh"
#include <cstring>

namespace {

using namespace st;
using namespace st::gemm;

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const OutMaps& tmC, const GemmParams& p,
                   cudaStream_t stream, int max_ctas) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, COMM_NONE>;
  static bool configured[st::kMaxDevices] = {false};   // the attribute is per device
  const int dev = st::current_device();
  if (!configured[dev]) {
    ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured[dev] = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
  int grid = tiles < st::sm_count() ? tiles : st::sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  GemmComm none{};
  kern<<<grid, NUM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, tmA, p, none);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

template <int BN, int STAGES>
int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const OutMaps& tmC,
                   const GemmParams& p, cudaStream_t stream, int max_ctas) {
  if (!a_mn && !b_mn) return launch_variant<BN, STAGES, false, false>(tmA, tmB, tmC, p, stream, max_ctas);
  if (!a_mn && b_mn) return launch_variant<BN, STAGES, false, true>(tmA, tmB, tmC, p, stream, max_ctas);
  if (a_mn && !b_mn) return launch_variant<BN, STAGES, true, false>(tmA, tmB, tmC, p, stream, max_ctas);
  return launch_variant<BN, STAGES, true, true>(tmA, tmB, tmC, p, stream, max_ctas);
}

}  // namespace

// Arguments of st_gemm_bf16 (plain C struct so that ctypes can build it).
struct StGemmArgs {
  const void* A;      // bf16
  const void* B;      // bf16
  void* C;            // bf16 or fp32
  const void* bias;   // bf16 [N] or null
  const void* residual;  // bf16 [M,N] or null
  void* aux_out;      // bf16 [M,N] or null: receives alpha*acc+bias before the activation
  const void* aux_in; // bf16 [M,N]: pre-activation for ACT_*_BWD
  long long lda, ldb, ldc, ldr, ld_aux_out, ld_aux_in;  // leading dimensions in elements
  long long batch_stride_a, batch_stride_b, batch_stride_c;  // elements (batch > 1)
  int M, N, K, batch;
  int a_mn_major, b_mn_major;
  int out_fp32, accumulate, act;
  float alpha;
  int max_ctas;  // 0 = one CTA per SM; >0 limits the grid (leaves SMs to concurrent kernels)
};

ST_API int st_gemm_bf16(const StGemmArgs* a, void* stream_v) {
  if (!a || !a->A || !a->B || !a->C) return st::fail(ST_ERR_INVALID, "gemm: null operand");
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0)
    return st::fail(ST_ERR_INVALID, "gemm: non-positive dimension");
  if ((a->lda & 7) || (a->ldb & 7))
    return st::fail(ST_ERR_INVALID, "gemm: lda/ldb must be multiples of 8 elements (16 bytes)");
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15))
    return st::fail(ST_ERR_INVALID, "gemm: A/B must be 16-byte aligned");
  if (a->batch > 1 && ((a->batch_stride_a & 7) || (a->batch_stride_b & 7)))
    return st::fail(ST_ERR_INVALID, "gemm: batch strides must be multiples of 8 elements");
  if ((a->act == ACT_GELU_BWD || a->act == ACT_RELU_BWD) && !a->aux_in)
    return st::fail(ST_ERR_INVALID, "gemm: backward activation needs aux_in");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);

  const bool small_n = a->N <= 128;
  const int BN = small_n ? 128 : 256;

  CUtensorMap tmA, tmB;
  {
    const uint64_t bsa = a->batch > 1 ? (uint64_t)a->batch_stride_a * 2 : (uint64_t)a->lda * 2 * (a->a_mn_major ? a->K : a->M);
    const uint64_t bsb = a->batch > 1 ? (uint64_t)a->batch_stride_b * 2 : (uint64_t)a->ldb * 2 * (a->b_mn_major ? a->K : a->N);
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a->a_mn_major) {
      dims[0] = a->K; dims[1] = a->M; box[0] = BK; box[1] = BM;
    } else {
      dims[0] = a->M; dims[1] = a->K; box[0] = 64; box[1] = BK;
    }
    dims[2] = a->batch; box[2] = 1;
    strides[0] = (uint64_t)a->lda * 2; strides[1] = bsa;
    if (!st::encode_tmap(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->A, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
    if (!a->b_mn_major) {
      dims[0] = a->K; dims[1] = a->N; box[0] = BK; box[1] = BN;
    } else {
      dims[0] = a->N; dims[1] = a->K; box[0] = 64; box[1] = BK;
    }
    strides[0] = (uint64_t)a->ldb * 2; strides[1] = bsb;
    if (!st::encode_tmap(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->B, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }

  GemmParams p{};  // zero-initialised: unset optional features (convolution geometry, epilogue operands) stay off
  p.C = a->C;
  p.ldc = a->ldc;
  p.bias = static_cast<const __nv_bfloat16*>(a->bias);
  p.residual = static_cast<const __nv_bfloat16*>(a->residual);
  p.ldr = a->ldr;
  p.aux_out = static_cast<__nv_bfloat16*>(a->aux_out);
  p.ld_aux_out = a->ld_aux_out;
  p.aux_in = static_cast<const __nv_bfloat16*>(a->aux_in);
  p.ld_aux_in = a->ld_aux_in;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.alpha = a->alpha;
  p.act = a->act;
  p.out_fp32 = a->out_fp32;
  p.accumulate = a->accumulate;
  p.batch = a->batch;
  p.batch_stride_c = a->batch_stride_c;
  p.err = st::error_word();
  p.use_tma_store = (!a->out_fp32 && !a->accumulate && (a->ldc & 7) == 0 &&
                     (reinterpret_cast<uintptr_t>(a->C) & 15) == 0 &&
                     (a->batch == 1 || (a->batch_stride_c & 7) == 0)) ? 1 : 0;
  OutMaps tmC;
  memset(&tmC, 0, sizeof(tmC));
  if (p.use_tma_store) {
    uint64_t dims[3] = {(uint64_t)a->N, (uint64_t)a->M, (uint64_t)a->batch};
    uint64_t strides[2] = {(uint64_t)a->ldc * 2,
                           a->batch > 1 ? (uint64_t)a->batch_stride_c * 2 : (uint64_t)a->ldc * 2 * a->M};
    uint32_t box[3] = {64, 32, 1};
    if (!st::encode_tmap(&tmC.m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->C, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }

  if (small_n)
    return dispatch_major<128, 6>(a->a_mn_major != 0, a->b_mn_major != 0, tmA, tmB, tmC, p, stream, a->max_ctas);
  return dispatch_major<256, 4>(a->a_mn_major != 0, a->b_mn_major != 0, tmA, tmB, tmC, p, stream, a->max_ctas);
}
