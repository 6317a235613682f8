// InfoNCE forward across ranks in ONE kernel: all-gather of the positive embeddings over
// NVLink + similarity GEMM (anchors · positivesᵀ / T) on tcgen05 + online row softmax.
//
// Every rank holds anchors A [R, D] and positives P [R, D] (rows L2-normalised by the caller,
// bf16, D a multiple of 64 up to 256).  The logits matrix is [R, W·R]; it is never written out.
//   * a few communication CTAs push this rank's positives into every rank's gather buffer
//     (multimem.st through NVSwitch, or peer stores) and publish one arrival flag per rank;
//   * compute CTA (m, g) owns 128 anchor rows and a group of 512 columns (= 4 tiles of 128
//     positives, all from one source rank): it waits (bounded) for that rank's flag — the local
//     rank's columns are read from the local shard without waiting —, runs the four
//     128x128xD MMAs with the accumulator in TMEM and folds each tile into a running
//     (max, sum-exp, positive-logit) per row;
//   * the partial statistics of the 2·W groups of a row block meet in global memory; the last
//     CTA to arrive combines them into the per-row log-sum-exp and loss.
// The gathered positives stay valid after the kernel (the backward GEMMs use them).
//
// Reference parity: info_nce_loss (crates/spiral-selfsup/src/contrastive.rs:96-153) is
// single-rank; the cross-rank negatives and the fusion are new.
#include "../common/host.h"
#include "comm.cuh"

struct StPeerGroup {
  int world, rank;
  unsigned epoch;
  unsigned long long signals[st::kMaxRanks];
  unsigned long long signals_mc;
};
namespace st {
void fill_peer_group(PeerGroup& g, const StPeerGroup& s);
}

namespace {
using namespace st;

constexpr int BLK = 128;
constexpr int TILES_PER_GROUP = 4;
constexpr int NUM_THREADS = 192;  // warps 0-3 softmax, warp 4 TMA, warp 5 MMA

struct NceParams {
  PeerGroup g;
  int R, D;                    // rows per rank, embedding width
  int slot_enter, slot_arrive;
  int compute_ctas;
  unsigned arrive_target;      // cumulative arrivals (communication CTAs x launches) per source rank
  const __nv_bfloat16* p_local;
  __nv_bfloat16* gather_peers[kMaxRanks];
  __nv_bfloat16* gather_mc;
  float scale_log2;            // (1/T) * log2(e)
  float* partial;              // [groups][R][3] (max2, sum, positive logit in log2 units)
  unsigned* counters;          // [R / 128]
  float* row_loss;             // [R]
  float* row_lse;              // [R] natural-log lse of the scaled logits
  unsigned* err;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int KB>  // D / 64
__global__ void __launch_bounds__(NUM_THREADS, 1)
info_nce_fwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmPg,
                    const __grid_constant__ CUtensorMap tmPl, const NceParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = p.g.world, Rk = p.g.rank;

  // ---------------------------- communication CTAs --------------------------------------
  if (static_cast<int>(blockIdx.x) >= p.compute_ctas) {
    __shared__ int s_ok;
    const int cta = blockIdx.x - p.compute_ctas, n_comm = gridDim.x - p.compute_ctas;
    if (threadIdx.x == 0) {
      bool ok = true;
      if (cta == 0) {
        fence_sys();
        for (int q = 0; q < W; ++q) st_relaxed_sys(p.g.signals[q] + p.slot_enter + Rk, p.g.epoch);
      }
      for (int q = 0; q < W && ok; ++q) ok = wait_flag_ge(p.g.signals[Rk] + p.slot_enter + q, p.g.epoch);
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) {
      if (threadIdx.x == 0) report_error(p.err, ERR_FLAG_TIMEOUT, 0xC700u);
      return;
    }
    const long long elems = (long long)p.R * p.D;
    const long long dst_off = (long long)Rk * elems;
    for (long long i = ((long long)cta * NUM_THREADS + threadIdx.x) * 8; i < elems;
         i += (long long)n_comm * NUM_THREADS * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(p.p_local + i);
      if (p.gather_mc) {
        multimem_st_v4(p.gather_mc + dst_off + i, v);
      } else {
        for (int q = 0; q < W; ++q) *reinterpret_cast<uint4*>(p.gather_peers[(Rk + q) % W] + dst_off + i) = v;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // every communication CTA counts itself in on each peer; the flag a consumer waits for is
      // "n_comm arrivals of this epoch", kept as a monotonically growing count
      fence_sys();
      for (int q = 0; q < W; ++q) red_release_sys_add(p.g.signals[(Rk + q) % W] + p.slot_arrive + Rk, 1u);
    }
    return;
  }

  // ---------------------------- compute CTAs --------------------------------------------
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) report_error(p.err, ERR_BOUNDS, 0xC701u);
    return;
  }
  constexpr int TILE = BLK * 64 * 2 * KB;          // bytes of a 128 x D operand tile
  uint8_t* sA = smem;
  uint8_t* sB = smem + TILE;                        // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * TILE);
  uint64_t* a_full = bars;
  uint64_t* b_full = bars + 1;     // 2
  uint64_t* b_empty = bars + 3;    // 2
  uint64_t* s_full = bars + 5;     // 2
  uint64_t* s_empty = bars + 7;    // 2 (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ int s_last;

  const int groups = (W * p.R) / (BLK * TILES_PER_GROUP);
  const int m_tile = blockIdx.x / groups;
  const int grp = blockIdx.x % groups;
  const int col0 = grp * BLK * TILES_PER_GROUP;     // first global column of this group
  const int src = col0 / p.R;                        // rank that owns these positives
  const int m0 = m_tile * BLK;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(a_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&b_full[i]), 1);
      mbar_init(smem_u32(&b_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      bool ok = true;
      const CUtensorMap* mapP = &tmPg;
      int row_base = col0;                           // row in the gathered [W*R, D] buffer
      if (src == Rk) {
        mapP = &tmPl;
        row_base = col0 - src * p.R;
      } else {
        // every communication CTA of the source rank adds one arrival per launch
        ok = wait_flag_ge(p.g.signals[Rk] + p.slot_arrive + src, p.arrive_target);
        if (!ok) {
          *abort_flag = 1;
          report_error(p.err, ERR_FLAG_TIMEOUT, 0xC702u);
        }
        fence_proxy_async_global();
      }
      if (ok) {
        mbar_arrive_expect_tx(smem_u32(a_full), TILE);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem_u32(sA + kb * (BLK * 128)), &tmA, smem_u32(a_full), kb * 64, m0);
        for (int t = 0; t < TILES_PER_GROUP; ++t) {
          const int st = t & 1;
          if (!mbar_wait(smem_u32(&b_empty[st]), ((t >> 1) & 1) ^ 1u, abort_flag)) break;
          mbar_arrive_expect_tx(smem_u32(&b_full[st]), TILE);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(smem_u32(sB + st * TILE + kb * (BLK * 128)), mapP, smem_u32(&b_full[st]), kb * 64,
                        row_base + t * BLK);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BLK, BLK, false, false);
      bool ok = mbar_wait(smem_u32(a_full), 0, abort_flag);
      for (int t = 0; t < TILES_PER_GROUP && ok; ++t) {
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(smem_u32(&s_empty[st]), ph ^ 1u, abort_flag)) break;
        if (!mbar_wait(smem_u32(&b_full[st]), ph, abort_flag)) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(sA), sb = smem_u32(sB + st * TILE);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + st * BLK, make_smem_desc_sw128(sa + kb * (BLK * 128) + k * 32, 16, 1024),
                         make_smem_desc_sw128(sb + kb * (BLK * 128) + k * 32, 16, 1024), idesc,
                         (kb | k) != 0 ? 1u : 0u);
        umma_commit(smem_u32(&s_full[st]));
        umma_commit(smem_u32(&b_empty[st]));
      }
    }
  } else {
    // ---- online softmax statistics: one thread per anchor row ----------------------------
    const int r = warp * 32 + lane;
    const int row_g = m0 + r;                                  // anchor row on this rank
    const int pos_col = Rk * p.R + row_g;                      // its positive's global column
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float m = -INFINITY, s = 0.0f, pos = 0.0f;
    bool ok = true;
    for (int t = 0; t < TILES_PER_GROUP; ++t) {
      const int st = t & 1;
      if (!mbar_wait_warp(smem_u32(&s_full[st]), (t >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int cbase = col0 + t * BLK;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_off + st * BLK + ch * 32, v);
        tmem_ld_wait();
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 32; ++c) mx = fmaxf(mx, __uint_as_float(v[c]));
        const float m_new = fmaxf(m, mx * p.scale_log2);
        s *= fast_exp2(m - m_new);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float z = __uint_as_float(v[c]) * p.scale_log2;
          s += fast_exp2(z - m_new);
          if (cbase + ch * 32 + c == pos_col) pos = z;
        }
        m = m_new;
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&s_empty[st]));
    }
    if (ok && row_g < p.R) {
      float* out = p.partial + ((long long)grp * p.R + row_g) * 3;
      out[0] = m;
      out[1] = s;
      out[2] = pos;
    }
  }

  tc_fence_before();
  __syncthreads();
  // ---- last CTA of the row block combines the groups ---------------------------------------
  if (!*abort_flag) {
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned prev = atomicAdd(p.counters + m_tile, 1u);
      s_last = (prev == static_cast<unsigned>(groups - 1)) ? 1 : 0;
      if (s_last) p.counters[m_tile] = 0;
    }
    __syncthreads();
    if (s_last && threadIdx.x < BLK) {
      __threadfence();
      const int row_g = m0 + threadIdx.x;
      if (row_g < p.R) {
        float m = -INFINITY, s = 0.0f, pos = 0.0f;
        for (int g2 = 0; g2 < groups; ++g2) {
          const volatile float* in = p.partial + ((long long)g2 * p.R + row_g) * 3;
          const float gm = in[0], gs = in[1];
          const float nm = fmaxf(m, gm);
          s = s * fast_exp2(m - nm) + gs * fast_exp2(gm - nm);
          m = nm;
          pos += in[2];
        }
        const float lse2 = m + log2f(s);
        p.row_lse[row_g] = lse2 * 0.6931471805599453f;
        p.row_loss[row_g] = (lse2 - pos) * 0.6931471805599453f;
      }
    }
  } else if (threadIdx.x == 0) {
    report_error(p.err, ERR_MBAR_TIMEOUT, 0xC703u);
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace

struct StInfoNceArgs {
  StPeerGroup g;
  unsigned long long anchors;                       // bf16 [R, D]
  unsigned long long positives;                     // bf16 [R, D] (this rank's shard)
  unsigned long long gather_peers[st::kMaxRanks];   // bf16 [W*R, D] on every rank
  unsigned long long gather_mc;
  unsigned long long partial;                       // fp32 [W*R/512][R][3] scratch
  unsigned long long counters;                      // u32 [R/128], zero before the first launch
  unsigned long long row_loss, row_lse;             // fp32 [R]
  int R, D;
  float inv_temperature;
  int slot_enter, slot_arrive;
  int comm_ctas;
  unsigned arrive_target;                           // cumulative arrivals expected per source rank
};

ST_API int st_info_nce_fwd(const StInfoNceArgs* a, void* stream_v) {
  if (!a) return st::fail(ST_ERR_INVALID, "info_nce: null args");
  const int W = a->g.world;
  if (W < 1 || W > st::kMaxRanks) return st::fail(ST_ERR_INVALID, "info_nce: bad world size");
  if (a->D % 64 != 0 || a->D > 256 || a->D <= 0) return st::fail(ST_ERR_INVALID, "info_nce: D must be 64, 128, 192 or 256");
  if (a->R % (BLK * TILES_PER_GROUP) != 0) return st::fail(ST_ERR_INVALID, "info_nce: rows per rank must be a multiple of 512");
  const int groups = (W * a->R) / (BLK * TILES_PER_GROUP);
  const int compute = (a->R / BLK) * groups;
  const int comm = a->comm_ctas < 1 ? 1 : a->comm_ctas;
  if (compute + comm > st::sm_count())
    return st::fail(ST_ERR_TOO_LARGE, "info_nce: problem needs more CTAs than SMs (all CTAs must be resident)");
  CUtensorMap tmA, tmPg, tmPl;
  if (!st::encode_tmap_2d_bf16(&tmA, reinterpret_cast<const void*>(a->anchors), a->D, a->R, (uint64_t)a->D * 2, 64, BLK) ||
      !st::encode_tmap_2d_bf16(&tmPg, reinterpret_cast<const void*>(a->gather_peers[a->g.rank]), a->D,
                               (uint64_t)W * a->R, (uint64_t)a->D * 2, 64, BLK) ||
      !st::encode_tmap_2d_bf16(&tmPl, reinterpret_cast<const void*>(a->positives), a->D, a->R, (uint64_t)a->D * 2, 64, BLK))
    return ST_ERR_CUDA;
  NceParams p;
  st::fill_peer_group(p.g, a->g);
  p.R = a->R; p.D = a->D;
  p.slot_enter = a->slot_enter; p.slot_arrive = a->slot_arrive;
  p.compute_ctas = compute;
  p.arrive_target = a->arrive_target;
  p.p_local = reinterpret_cast<const __nv_bfloat16*>(a->positives);
  for (int i = 0; i < st::kMaxRanks; ++i) p.gather_peers[i] = reinterpret_cast<__nv_bfloat16*>(a->gather_peers[i]);
  p.gather_mc = reinterpret_cast<__nv_bfloat16*>(a->gather_mc);
  p.scale_log2 = a->inv_temperature * 1.4426950408889634f;
  p.partial = reinterpret_cast<float*>(a->partial);
  p.counters = reinterpret_cast<unsigned*>(a->counters);
  p.row_loss = reinterpret_cast<float*>(a->row_loss);
  p.row_lse = reinterpret_cast<float*>(a->row_lse);
  p.err = st::error_word();
  const int KB = a->D / 64;
  const int smem = 3 * (BLK * 64 * 2 * KB) + 256;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  auto launch = [&](auto kern) -> int {
    ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<compute + comm, NUM_THREADS, smem, s>>>(tmA, tmPg, tmPl, p);
    ST_CUDA_CHECK(cudaGetLastError());
    return ST_OK;
  };
  switch (KB) {
    case 1: return launch(info_nce_fwd_kernel<1>);
    case 2: return launch(info_nce_fwd_kernel<2>);
    case 3: return launch(info_nce_fwd_kernel<3>);
    default: return launch(info_nce_fwd_kernel<4>);
  }
}

// ---- backward helper: d_logits = (exp(logit - lse) - onehot) * coef, bf16, in both orientations ---------------------
// The two gradient GEMMs want d_logits as [R, C] (for d_anchor = d_logits @ P) and as [C, R] (rows = the gathered
// positives, for the GEMM -> reduce-scatter of d_positives).  One pass over the fp32 logits writes both: a 32 x 32
// tile goes through shared memory so that both stores are coalesced.
namespace {

__global__ void info_nce_grad_kernel(const float* __restrict__ logits, const float* __restrict__ row_lse,
                                     const float* __restrict__ coef, __nv_bfloat16* __restrict__ dl,
                                     __nv_bfloat16* __restrict__ dl_t, int R, int C, int target_offset) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const float k = coef[0];
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    float v = 0.0f;
    if (r < R && c < C) {
      v = __expf(logits[(long long)r * C + c] - row_lse[r]);
      if (c == r + target_offset) v -= 1.0f;
      v *= k;
      dl[(long long)r * C + c] = __float2bfloat16(v);
    }
    tile[i][threadIdx.x] = v;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < R && c < C) dl_t[(long long)c * R + r] = __float2bfloat16(tile[threadIdx.x][i]);
  }
}

}  // namespace

// logits [R, C] fp32 (already divided by the temperature), row_lse [R], coef: one device float (upstream gradient / R);
// the positive of row r is column r + target_offset.  Writes dl [R, C] and dl_t [C, R] in bf16.
ST_API int st_info_nce_grad(const float* logits, const float* row_lse, const float* coef, void* dl, void* dl_t, int R,
                            int C, int target_offset, void* stream_v) {
  if (R <= 0 || C <= 0) return st::fail(ST_ERR_INVALID, "info_nce_grad: empty problem");
  if (target_offset < 0 || target_offset + R > C) return st::fail(ST_ERR_INVALID, "info_nce_grad: positives fall outside the columns");
  dim3 grid((C + 31) / 32, (R + 31) / 32), block(32, 8);
  info_nce_grad_kernel<<<grid, block, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      logits, row_lse, coef, reinterpret_cast<__nv_bfloat16*>(dl), reinterpret_cast<__nv_bfloat16*>(dl_t), R, C, target_offset);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
