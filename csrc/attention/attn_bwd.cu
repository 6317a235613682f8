// Attention backward (dQ, dK, dV) on sm_100a tensor cores.
//
// Three launches:
//   1. delta[b,h,s] = sum_d O·dO                          (one warp per row)
//   2. main kernel: one CTA owns a 128-row KV tile of one (batch, head) and walks the query
//      tiles that attend to it.  Per query tile, five tcgen05 GEMMs:
//          S  = Q·Kᵀ, dP = dO·Vᵀ                (TMEM, fp32)
//          P  = exp2(S·c − lse), dS = P∘(dP − delta)   (registers → bf16 in shared memory)
//          dV += Pᵀ·dO, dK += dSᵀ·Q             (TMEM accumulators that live across tiles)
//          dQ_tile = dS·K                       (TMEM, reusing the S columns)
//      Pᵀ and dSᵀ need no transposition pass: the bytes written for the K-major operand
//      (rows = queries) are read again through an MN-major descriptor.  dQ tiles are added to
//      an fp32 accumulator in global memory with vector atomics (several KV tiles
//      contribute to each query tile).
//   3. dQ accumulator → bf16, scaled.
// Warp 8 is the TMA producer (K, V once; Q and dO through a 3-slot ring), warp 9 issues the
// MMAs and owns TMEM, warps 0-7 do the element-wise work with two threads per row.
//
// The reference has no attention backward; the oracle is PyTorch autograd of the fp32 math.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace st {
bool encode_bshd_tmap(CUtensorMap* out, const void* base, int B, int S, int H, int D,
                      long long sb, long long ss, long long sh, int box_rows);
}

namespace {
using namespace st;

constexpr int BLK = 128;
constexpr int NUM_THREADS = 320;

struct AttnBwdParams {
  const float* lse;
  const float* delta;
  float* dq_acc;               // [B,H,Sq,D] fp32
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
  int B, H, Sq, Sk;
  float scale, scale_log2;
  int causal;
  unsigned* err;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct BwdSmem {
  static constexpr int TILE = BLK * D * 2;
  static constexpr int P_TILE = BLK * BLK * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + TILE;
  static constexpr int RING_OFF = V_OFF + TILE;      // 3 slots
  static constexpr int P_OFF = RING_OFF + 3 * TILE;
  static constexpr int DS_OFF = P_OFF + P_TILE;
  static constexpr int BAR_OFF = DS_OFF + P_TILE;
  static constexpr int TOTAL = BAR_OFF + 256;
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DH = D / 2;
  constexpr int KB = D / 64;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 384, DQ_COL = 0;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) report_error(p.err, ERR_BOUNDS, 0xA7B1u);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;           // 1
  uint64_t* ring_full = bars + 1;     // 3
  uint64_t* ring_empty = bars + 4;    // 3
  uint64_t* sdp_full = bars + 7;      // 1
  uint64_t* pds_full = bars + 8;      // 1 (256 arrivals)
  uint64_t* dq_full = bars + 9;       // 1
  uint64_t* dq_read = bars + 10;      // 1 (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kv0 = j * BLK;
  const int n_q = (p.Sq + BLK - 1) / BLK;
  const int i_start = p.causal ? j : 0;
  const int n_iter = n_q - i_start;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(kv_full), 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(smem_u32(&ring_full[s]), 1);
      mbar_init(smem_u32(&ring_empty[s]), 1);
    }
    mbar_init(smem_u32(sdp_full), 1);
    mbar_init(smem_u32(pds_full), 256);
    mbar_init(smem_u32(dq_full), 1);
    mbar_init(smem_u32(dq_read), 256);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------------------- TMA producer -----------------------------------------
    if (lane == 0 && n_iter > 0) {
      const uint32_t kvb = smem_u32(kv_full);
      mbar_arrive_expect_tx(kvb, 2 * L::TILE);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        tma_load_4d(smem_u32(smem + L::K_OFF + kb * (BLK * 128)), &tmK, kvb, kb * 64, h, kv0, b);
        tma_load_4d(smem_u32(smem + L::V_OFF + kb * (BLK * 128)), &tmV, kvb, kb * 64, h, kv0, b);
      }
      for (int seq = 0; seq < 2 * n_iter; ++seq) {
        const int slot = seq % 3;
        const uint32_t ph = (seq / 3) & 1;
        if (!mbar_wait(smem_u32(&ring_empty[slot]), ph ^ 1u, abort_flag)) break;
        const uint32_t fb = smem_u32(&ring_full[slot]);
        mbar_arrive_expect_tx(fb, L::TILE);
        const int q0 = (i_start + (seq >> 1)) * BLK;
        const CUtensorMap* tm = (seq & 1) ? &tmdO : &tmQ;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(smem_u32(smem + L::RING_OFF + slot * L::TILE + kb * (BLK * 128)), tm, fb,
                      kb * 64, h, q0, b);
      }
    }
  } else if (warp == 9) {
    // ---------------------------- MMA issuer -------------------------------------------
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);   // S, dP
      constexpr uint32_t idesc_t = make_idesc_bf16(BLK, D, true, true);       // dV, dK
      constexpr uint32_t idesc_q = make_idesc_bf16(BLK, D, false, true);      // dQ
      const uint32_t sk = smem_u32(smem + L::K_OFF);
      const uint32_t sv = smem_u32(smem + L::V_OFF);
      const uint32_t sp = smem_u32(smem + L::P_OFF);
      const uint32_t sds = smem_u32(smem + L::DS_OFF);
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag);
      for (int n = 0; n < n_iter && ok; ++n) {
        const int slot_q = (2 * n) % 3, slot_o = (2 * n + 1) % 3;
        const uint32_t ph_q = ((2 * n) / 3) & 1, ph_o = ((2 * n + 1) / 3) & 1;
        const uint32_t sq = smem_u32(smem + L::RING_OFF + slot_q * L::TILE);
        const uint32_t sdo = smem_u32(smem + L::RING_OFF + slot_o * L::TILE);
        if (n > 0 && !mbar_wait(smem_u32(dq_read), (n - 1) & 1, abort_flag)) break;
        if (!mbar_wait(smem_u32(&ring_full[slot_q]), ph_q, abort_flag)) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + S_COL,
                         make_smem_desc_sw128(sq + kb * (BLK * 128) + k * 32, 16, 1024),
                         make_smem_desc_sw128(sk + kb * (BLK * 128) + k * 32, 16, 1024), idesc_s,
                         (kb | k) != 0 ? 1u : 0u);
        if (!mbar_wait(smem_u32(&ring_full[slot_o]), ph_o, abort_flag)) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + DP_COL,
                         make_smem_desc_sw128(sdo + kb * (BLK * 128) + k * 32, 16, 1024),
                         make_smem_desc_sw128(sv + kb * (BLK * 128) + k * 32, 16, 1024), idesc_s,
                         (kb | k) != 0 ? 1u : 0u);
        umma_commit(smem_u32(sdp_full));

        if (!mbar_wait(smem_u32(pds_full), n & 1, abort_flag)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {
          // dV[kv, d] += sum_q P[q, kv] dO[q, d]
          umma_bf16_ss(tmem_base + DV_COL,
                       make_smem_desc_sw128(sp + kk * (16 * 128), BLK * 128, 1024),
                       make_smem_desc_sw128(sdo + kk * (16 * 128), BLK * 128, 1024), idesc_t,
                       (n | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {
          // dK[kv, d] += sum_q dS[q, kv] Q[q, d]
          umma_bf16_ss(tmem_base + DK_COL,
                       make_smem_desc_sw128(sds + kk * (16 * 128), BLK * 128, 1024),
                       make_smem_desc_sw128(sq + kk * (16 * 128), BLK * 128, 1024), idesc_t,
                       (n | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {
          // dQ[q, d] = sum_kv dS[q, kv] K[kv, d]
          umma_bf16_ss(tmem_base + DQ_COL,
                       make_smem_desc_sw128(sds + (kk >> 2) * (BLK * 128) + (kk & 3) * 32, 16, 1024),
                       make_smem_desc_sw128(sk + kk * (16 * 128), BLK * 128, 1024), idesc_q,
                       kk != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(dq_full));
        umma_commit(smem_u32(&ring_empty[slot_q]));
        umma_commit(smem_u32(&ring_empty[slot_o]));
      }
    }
  } else {
    // ---------------------------- element-wise warps -----------------------------------
    const int quad = warp & 3;
    const int half = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    for (int n = 0; n < n_iter; ++n) {
      const int i = i_start + n;
      const int row_g = i * BLK + r;
      const bool row_ok = row_g < p.Sq;
      const long long stat_idx = ((long long)b * p.H + h) * p.Sq + row_g;
      const float lse2 = row_ok ? p.lse[stat_idx] * LOG2E : 0.0f;
      const float dlt = row_ok ? p.delta[stat_idx] : 0.0f;
      if (!mbar_wait_warp(smem_u32(sdp_full), n & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && (i == j);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t s_r[32], dp_r[32];
        tmem_ld_32x32(tmem_base + lane_off + S_COL + half * 64 + ch * 32, s_r);
        tmem_ld_32x32(tmem_base + lane_off + DP_COL + half * 64 + ch * 32, dp_r);
        tmem_ld_wait();
        const int colbase = half * 64 + ch * 32;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float pv[8], dsv[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int cl = colbase + c8 * 8 + q;        // column inside the KV tile
            const int colg = kv0 + cl;
            const bool dead = !row_ok || colg >= p.Sk || (diag && colg > row_g);
            const float pe = dead ? 0.0f
                                  : fast_exp2(__uint_as_float(s_r[c8 * 8 + q]) * p.scale_log2 - lse2);
            pv[q] = pe;
            dsv[q] = pe * (__uint_as_float(dp_r[c8 * 8 + q]) - dlt);
          }
          uint4 up, ud;
          up.x = pack_bf16x2(pv[0], pv[1]); up.y = pack_bf16x2(pv[2], pv[3]);
          up.z = pack_bf16x2(pv[4], pv[5]); up.w = pack_bf16x2(pv[6], pv[7]);
          ud.x = pack_bf16x2(dsv[0], dsv[1]); ud.y = pack_bf16x2(dsv[2], dsv[3]);
          ud.z = pack_bf16x2(dsv[4], dsv[5]); ud.w = pack_bf16x2(dsv[6], dsv[7]);
          const uint32_t off = half * (BLK * 128) + sw128_offset(r, ch * 4 + c8);
          *reinterpret_cast<uint4*>(smem + L::P_OFF + off) = up;
          *reinterpret_cast<uint4*>(smem + L::DS_OFF + off) = ud;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(pds_full));

      if (!mbar_wait_warp(smem_u32(dq_full), n & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = p.dq_acc + (((long long)b * p.H + h) * p.Sq + row_g) * D + half * DH;
#pragma unroll
      for (int ch = 0; ch < DH / 32; ++ch) {
        uint32_t t[32];
        tmem_ld_32x32(tmem_base + lane_off + DQ_COL + half * DH + ch * 32, t);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float4 v = make_float4(__uint_as_float(t[q * 4]), __uint_as_float(t[q * 4 + 1]),
                                   __uint_as_float(t[q * 4 + 2]), __uint_as_float(t[q * 4 + 3]));
            atomicAdd(reinterpret_cast<float4*>(dq_row + ch * 32 + q * 4), v);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(dq_read));
    }
    if (ok && n_iter > 0) {
      // dq_full of the last iteration also covers every dV / dK MMA
      const int kv_row = kv0 + r;
      const bool kv_ok = kv_row < p.Sk;
      __nv_bfloat16* dvp = p.dV + (long long)b * p.dv_sb + (long long)kv_row * p.dv_ss +
                           (long long)h * p.dv_sh + half * DH;
      __nv_bfloat16* dkp = p.dK + (long long)b * p.dk_sb + (long long)kv_row * p.dk_ss +
                           (long long)h * p.dk_sh + half * DH;
#pragma unroll
      for (int ch = 0; ch < DH / 32; ++ch) {
        // TMEM loads are warp-collective: every lane issues them, only the stores are predicated
        uint32_t tv[32], tk[32];
        tmem_ld_32x32(tmem_base + lane_off + DV_COL + half * DH + ch * 32, tv);
        tmem_ld_32x32(tmem_base + lane_off + DK_COL + half * DH + ch * 32, tk);
        tmem_ld_wait();
        if (kv_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 uv, uk;
            uv.x = pack_bf16x2(__uint_as_float(tv[q * 8 + 0]), __uint_as_float(tv[q * 8 + 1]));
            uv.y = pack_bf16x2(__uint_as_float(tv[q * 8 + 2]), __uint_as_float(tv[q * 8 + 3]));
            uv.z = pack_bf16x2(__uint_as_float(tv[q * 8 + 4]), __uint_as_float(tv[q * 8 + 5]));
            uv.w = pack_bf16x2(__uint_as_float(tv[q * 8 + 6]), __uint_as_float(tv[q * 8 + 7]));
            uk.x = pack_bf16x2(__uint_as_float(tk[q * 8 + 0]) * p.scale, __uint_as_float(tk[q * 8 + 1]) * p.scale);
            uk.y = pack_bf16x2(__uint_as_float(tk[q * 8 + 2]) * p.scale, __uint_as_float(tk[q * 8 + 3]) * p.scale);
            uk.z = pack_bf16x2(__uint_as_float(tk[q * 8 + 4]) * p.scale, __uint_as_float(tk[q * 8 + 5]) * p.scale);
            uk.w = pack_bf16x2(__uint_as_float(tk[q * 8 + 6]) * p.scale, __uint_as_float(tk[q * 8 + 7]) * p.scale);
            reinterpret_cast<uint4*>(dvp + ch * 32)[q] = uv;
            reinterpret_cast<uint4*>(dkp + ch * 32)[q] = uk;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_error(p.err, ERR_MBAR_TIMEOUT, 0xA7B0u);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d]; one warp per (b,s,h).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, int B, int S, int H, int D,
                                  long long o_sb, long long o_ss, long long o_sh, long long do_sb,
                                  long long do_ss, long long do_sh) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (w >= total) return;
  const int hh = w % H;
  const long long bs = w / H;
  const int s = bs % S;
  const int bb = bs / S;
  const __nv_bfloat16* op = O + bb * o_sb + s * o_ss + hh * o_sh;
  const __nv_bfloat16* dp = dO + bb * do_sb + s * do_ss + hh * do_sh;
  float acc = 0.0f;
  for (int c = lane * 2; c < D; c += 64) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + c));
    float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + c));
    acc += a.x * g.x + a.y * g.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[((long long)bb * H + hh) * S + s] = acc;
}

// dQ[b,s,h,:] = bf16(scale * dq_acc[b,h,s,:])
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dQ,
                                       int B, int S, int H, int D, long long sb, long long ss,
                                       long long sh, float scale) {
  const int vec = D / 4;
  const long long total = (long long)B * H * S * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = i % vec;
    const long long row = i / vec;
    const int s = row % S;
    const long long bh = row / S;
    const int hh = bh % H;
    const int bb = bh / H;
    const float4 a = reinterpret_cast<const float4*>(acc)[i];
    uint2 u;
    u.x = pack_bf16x2(a.x * scale, a.y * scale);
    u.y = pack_bf16x2(a.z * scale, a.w * scale);
    *reinterpret_cast<uint2*>(dQ + bb * sb + s * ss + hh * sh + v * 4) = u;
  }
}

}  // namespace

struct StAttnBwdArgs {
  const void* Q; const void* K; const void* V; const void* O; const void* dO;
  const float* lse; float* delta; float* dQ_acc;
  void* dQ; void* dK; void* dV;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh;
  long long do_sb, do_ss, do_sh, dq_sb, dq_ss, dq_sh, dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
  int B, H, Sq, Sk, D;
  float scale;
  int causal;
};

// delta: fp32 [B,H,Sq] workspace; dQ_acc: fp32 [B,H,Sq,D] workspace that must be ZERO on entry.
ST_API int st_attn_bwd(const StAttnBwdArgs* a, void* stream_v) {
  if (!a || !a->Q || !a->K || !a->V || !a->O || !a->dO || !a->lse || !a->delta || !a->dQ_acc ||
      !a->dQ || !a->dK || !a->dV)
    return st::fail(ST_ERR_INVALID, "attn_bwd: null pointer");
  if (a->D != 64 && a->D != 128) return st::fail(ST_ERR_INVALID, "attn_bwd: head_dim must be 64 or 128");
  if (a->causal && a->Sq != a->Sk) return st::fail(ST_ERR_INVALID, "attn_bwd: causal needs seq_q == seq_k");
  const long long strides[] = {a->q_sb, a->q_ss, a->q_sh, a->k_sb, a->k_ss, a->k_sh, a->v_sb, a->v_ss,
                               a->v_sh, a->o_sb, a->o_ss, a->o_sh, a->do_sb, a->do_ss, a->do_sh,
                               a->dq_sb, a->dq_ss, a->dq_sh, a->dk_sb, a->dk_ss, a->dk_sh,
                               a->dv_sb, a->dv_ss, a->dv_sh};
  for (long long s : strides)
    if (s & 7) return st::fail(ST_ERR_INVALID, "attn_bwd: strides must be multiples of 8 elements");
  const void* ptrs[] = {a->Q, a->K, a->V, a->O, a->dO, a->dQ, a->dK, a->dV, a->dQ_acc};
  for (const void* q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) & 15) return st::fail(ST_ERR_INVALID, "attn_bwd: pointers must be 16-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);

  {
    const long long warps = (long long)a->B * a->Sq * a->H;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(a->O), static_cast<const __nv_bfloat16*>(a->dO), a->delta,
        a->B, a->Sq, a->H, a->D, a->o_sb, a->o_ss, a->o_sh, a->do_sb, a->do_ss, a->do_sh);
    ST_CUDA_CHECK(cudaGetLastError());
  }

  CUtensorMap tq, tk, tv, tdo;
  if (!st::encode_bshd_tmap(&tq, a->Q, a->B, a->Sq, a->H, a->D, a->q_sb, a->q_ss, a->q_sh, BLK) ||
      !st::encode_bshd_tmap(&tk, a->K, a->B, a->Sk, a->H, a->D, a->k_sb, a->k_ss, a->k_sh, BLK) ||
      !st::encode_bshd_tmap(&tv, a->V, a->B, a->Sk, a->H, a->D, a->v_sb, a->v_ss, a->v_sh, BLK) ||
      !st::encode_bshd_tmap(&tdo, a->dO, a->B, a->Sq, a->H, a->D, a->do_sb, a->do_ss, a->do_sh, BLK))
    return ST_ERR_CUDA;
  AttnBwdParams p;
  p.lse = a->lse; p.delta = a->delta; p.dq_acc = a->dQ_acc;
  p.dK = static_cast<__nv_bfloat16*>(a->dK);
  p.dV = static_cast<__nv_bfloat16*>(a->dV);
  p.dk_sb = a->dk_sb; p.dk_ss = a->dk_ss; p.dk_sh = a->dk_sh;
  p.dv_sb = a->dv_sb; p.dv_ss = a->dv_ss; p.dv_sh = a->dv_sh;
  p.B = a->B; p.H = a->H; p.Sq = a->Sq; p.Sk = a->Sk;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.causal = a->causal;
  p.err = st::error_word();
  dim3 grid((a->Sk + BLK - 1) / BLK, a->H, a->B);
  if (a->D == 128) {
    static bool cfg = false;
    if (!cfg) {
      ST_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<128>::TOTAL));
      cfg = true;
    }
    attn_bwd_kernel<128><<<grid, NUM_THREADS, BwdSmem<128>::TOTAL, s>>>(tq, tk, tv, tdo, p);
  } else {
    static bool cfg = false;
    if (!cfg) {
      ST_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<64>::TOTAL));
      cfg = true;
    }
    attn_bwd_kernel<64><<<grid, NUM_THREADS, BwdSmem<64>::TOTAL, s>>>(tq, tk, tv, tdo, p);
  }
  ST_CUDA_CHECK(cudaGetLastError());
  {
    const long long total = (long long)a->B * a->H * a->Sq * (a->D / 4);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_dq_convert_kernel<<<(unsigned)blocks, 256, 0, s>>>(a->dQ_acc, static_cast<__nv_bfloat16*>(a->dQ),
                                                           a->B, a->Sq, a->H, a->D, a->dq_sb, a->dq_ss,
                                                           a->dq_sh, a->scale);
    ST_CUDA_CHECK(cudaGetLastError());
  }
  return ST_OK;
}
