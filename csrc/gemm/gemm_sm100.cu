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
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {

using namespace st;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_GELU_BWD = 3, ACT_RELU_BWD = 4 };

struct GemmParams {
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* aux_out;
  long long ld_aux_out;
  const __nv_bfloat16* aux_in;
  long long ld_aux_in;
  int M, N, K;
  float alpha;
  int act;
  int out_fp32;
  int accumulate;
  int batch;             // number of independent problems (grid-strided together)
  long long batch_stride_c;  // elements
  unsigned* err;
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  // groups of 8 M-tiles share the same B tiles while they are L2-resident
  constexpr int GM = 8;
  const int group_size = GM * tiles_n;
  const int g = t / group_size;
  const int first_m = g * GM;
  const int gm = min(GM, tiles_m - first_m);
  const int r = t - g * group_size;
  tm = first_m + r % gm;
  tn = r / gm;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = tiles_m * tiles_n;
  const int total_tiles = tiles_per_batch * p.batch;
  const int k_blocks = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                 : (2 * BN <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tfull_bar[a]), 1);
      mbar_init(smem_u32(&tempty_bar[a]), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int b = t / tiles_per_batch;
        int tm, tn;
        tile_coords(t - b * tiles_per_batch, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_arrive_expect_tx(fb, L::STAGE_BYTES);
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_3d(sa, &tmA, fb, k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * (64 * BK * 2), &tmA, fb, m0 + 64 * j, k0, b);
          }
          if constexpr (!B_MN) {
            tma_load_3d(sb, &tmB, fb, k0, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (64 * BK * 2), &tmB, fb, n0 + 64 * j, k0, b);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da, db;
            if constexpr (!A_MN)
              da = make_smem_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024);
            else
              da = make_smem_desc_sw128(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            if constexpr (!B_MN)
              db = make_smem_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024);
            else
              db = make_smem_desc_sw128(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            umma_bf16_ss(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // frees the smem stage when MMAs finish
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(smem_u32(&tfull_bar[acc]));
      }
    }
  } else {
    // ------------------------------- epilogue warps -----------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int iter = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++iter) {
      const int b = t / tiles_per_batch;
      int tm, tn;
      tile_coords(t - b * tiles_per_batch, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait_warp(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const long long c_base = (long long)b * p.batch_stride_c + (long long)row * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const bool full = (col0 + 32 <= p.N);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (full || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
        }
        if (p.aux_out) {
          __nv_bfloat16* a = p.aux_out + (long long)row * p.ld_aux_out + col0;
          if (full && (p.ld_aux_out & 7) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              reinterpret_cast<uint4*>(a)[q] = u;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) a[j] = __float2bfloat16(v[j]);
          }
        }
        if (p.act == ACT_RELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
        } else if (p.act == ACT_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        } else if (p.act == ACT_GELU_BWD || p.act == ACT_RELU_BWD) {
          const __nv_bfloat16* a = p.aux_in + (long long)row * p.ld_aux_in + col0;
          float x[32];
          if (full && (p.ld_aux_in & 7) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u = reinterpret_cast<const uint4*>(a)[q];
              float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                     f3 = unpack_bf16x2(u.w);
              x[q * 8 + 0] = f0.x; x[q * 8 + 1] = f0.y; x[q * 8 + 2] = f1.x; x[q * 8 + 3] = f1.y;
              x[q * 8 + 4] = f2.x; x[q * 8 + 5] = f2.y; x[q * 8 + 6] = f3.x; x[q * 8 + 7] = f3.y;
            }
          } else {
            for (int j = 0; j < 32; ++j) x[j] = (col0 + j < p.N) ? __bfloat162float(a[j]) : 0.0f;
          }
          if (p.act == ACT_GELU_BWD) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= gelu_tanh_grad(x[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = x[j] > 0.0f ? v[j] : 0.0f;
          }
        }
        if (p.residual) {
          const __nv_bfloat16* rs = p.residual + (long long)row * p.ldr + col0;
          if (full && (p.ldr & 7) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u = reinterpret_cast<const uint4*>(rs)[q];
              float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                     f3 = unpack_bf16x2(u.w);
              v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
              v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += __bfloat162float(rs[j]);
          }
        }
        if (p.out_fp32) {
          float* cp = reinterpret_cast<float*>(p.C) + c_base + col0;
          if (full && (p.ldc & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (p.accumulate) {
                float4 old = reinterpret_cast<float4*>(cp)[q];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              reinterpret_cast<float4*>(cp)[q] = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) cp[j] = p.accumulate ? cp[j] + v[j] : v[j];
          }
        } else {
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + c_base + col0;
          if (full && (p.ldc & 7) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (p.accumulate) {
                uint4 u = reinterpret_cast<const uint4*>(cp)[q];
                float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                       f3 = unpack_bf16x2(u.w);
                v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
                v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
              }
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              reinterpret_cast<uint4*>(cp)[q] = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) {
                float o = v[j];
                if (p.accumulate) o += __bfloat162float(cp[j]);
                cp[j] = __float2bfloat16(o);
              }
          }
        }
      }
      // hand the accumulator back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
    }
  }

  // ------------------------------- teardown -------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_error(p.err, ERR_MBAR_TIMEOUT, 0x6E00u);
    // give copies that are still in flight a bounded time to land before smem is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                   cudaStream_t stream, int max_ctas) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
  int grid = tiles < st::sm_count() ? tiles : st::sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kern<<<grid, NUM_THREADS, L::TOTAL, stream>>>(tmA, tmB, p);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

template <int BN, int STAGES>
int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                   const GemmParams& p, cudaStream_t stream, int max_ctas) {
  if (!a_mn && !b_mn) return launch_variant<BN, STAGES, false, false>(tmA, tmB, p, stream, max_ctas);
  if (!a_mn && b_mn) return launch_variant<BN, STAGES, false, true>(tmA, tmB, p, stream, max_ctas);
  if (a_mn && !b_mn) return launch_variant<BN, STAGES, true, false>(tmA, tmB, p, stream, max_ctas);
  return launch_variant<BN, STAGES, true, true>(tmA, tmB, p, stream, max_ctas);
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

  GemmParams p;
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

  if (small_n)
    return dispatch_major<128, 6>(a->a_mn_major != 0, a->b_mn_major != 0, tmA, tmB, p, stream, a->max_ctas);
  return dispatch_major<256, 4>(a->a_mn_major != 0, a->b_mn_major != 0, tmA, tmB, p, stream, a->max_ctas);
}
