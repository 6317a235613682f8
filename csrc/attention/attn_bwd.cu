// Attention backward (dQ, dK, dV) on sm_100a tensor cores.
//
// Three launches:
//   1. delta[b,h,s] = sum_d O·dO                          (one warp per row)
//   2. dK/dV pass (MODE_KV): one CTA owns a 128-row KV tile of one (batch, head) and walks the
//      query tiles that attend to it.  Per query tile, four tcgen05 GEMMs:
//          S  = Q·Kᵀ, dP = dO·Vᵀ                          (TMEM, fp32)
//          P  = exp2(S·c − lse), dS = P∘(dP − delta)      (registers → bf16 in shared memory)
//          dK += dSᵀ·Q, dV += Pᵀ·dO                       (TMEM accumulators that live across tiles)
//      Pᵀ and dSᵀ need no transposition pass: the bytes written for the K-major operand
//      (rows = queries) are read again through an MN-major descriptor.
//   3. dQ pass (MODE_Q): one CTA owns a 128-row query tile and walks the KV tiles it attends to:
//          S, dP as above; dS → shared memory; dQ += dS·K  (TMEM accumulator across KV tiles)
//      and writes dQ once, scaled, as bf16.
// Recomputing S and dP in the dQ pass costs two extra GEMMs per tile pair, but it removes the
// fp32 dQ accumulator in global memory with its 64 KB of vector atomics per tile pair, the
// conversion pass and the zero fill, and — because no pass needs more than 512 TMEM columns
// minus one operand — lets both passes software-pipeline: the element-wise phase is split in
// two (P from S, then dS from dP), S of the next tile is issued as soon as this tile's S has
// been read, and dP of the next tile right after this tile's accumulate GEMMs, so the tensor
// pipe works while the element-wise warps do.
// Warp 16 is the TMA producer (two stationary tiles once; the streamed pair through a ring),
// warp 17 issues the MMAs and owns TMEM, warps 0-15 do the element-wise work with four threads
// per row (with two, the element-wise phase was latency-bound: 2 warps per scheduler cannot hide
// the TMEM-load and MUFU latencies).
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
constexpr int EW_WARPS = 16;                       // element-wise warps: four threads per row, 32 key columns each
constexpr int EW_THREADS = EW_WARPS * 32;
constexpr int NUM_THREADS = EW_THREADS + 64;       // + TMA producer warp + MMA warp
constexpr int MODE_KV = 0, MODE_Q = 1;

struct AttnBwdParams {
  const float* lse;
  const float* delta;
  __nv_bfloat16* dQ;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long dq_sb, dq_ss, dq_sh, dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
  int B, H, Sq, Sk;
  float scale, scale_log2;
  int causal;
  unsigned* err;
  // optional additive biases and valid lengths, as in the forward kernel (null = absent)
  const float* key_bias;
  const float* attn_bias;
  const int* lengths;
  long long kb_sb, kb_sh, ab_sb, ab_sh, ab_sq;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, int MODE>
struct BwdSmem {
  static constexpr int TILE = BLK * D * 2;
  static constexpr int P_TILE = BLK * BLK * 2;
  // streamed tiles: stream A is Q (dK/dV pass) or K (dQ pass), stream B is dO or V.  The A tile is read by
  // the first GEMM of an iteration (S) and by the last one (dK or dQ), so it lives for more than a whole
  // iteration; the B tile is released early (after dV, or right after dP in the dQ pass).  The dK/dV pass
  // has room for three streamed tiles next to K, V, P and dS: two A, one B.  The dQ pass has no P buffer:
  // three A (with two, the issuer measured 0.47 us per iteration waiting for K), one B.
  static constexpr int NA = MODE == MODE_KV ? 2 : 3;
  static constexpr int NB = 1;
  static constexpr int STAT0_OFF = 0;                  // K (MODE_KV) or Q (MODE_Q)
  static constexpr int STAT1_OFF = STAT0_OFF + TILE;   // V (MODE_KV) or dO (MODE_Q)
  static constexpr int A_OFF = STAT1_OFF + TILE;
  static constexpr int B_OFF = A_OFF + NA * TILE;
  static constexpr int DS_OFF = B_OFF + NB * TILE;
  static constexpr int P_OFF = DS_OFF + P_TILE;        // MODE_KV only
  static constexpr int BAR_OFF = P_OFF + (MODE == MODE_KV ? P_TILE : 0);
  static constexpr int TOTAL = BAR_OFF + 256;
};

// 16 bytes of eight values → bf16, written at the swizzled position of (row r, 16-byte chunk c16)
__device__ __forceinline__ void store8_bf16(uint8_t* tile, int r, int c16, const float* v) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(tile + sw128_offset(r, c16)) = u;
}

template <int D, int MODE, bool BIAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdParams p) {
  using L = BwdSmem<D, MODE>;
  constexpr int KB = D / 64;
  constexpr int NA = L::NA, NB = L::NB;
  // TMEM columns.  MODE_KV: S, dP, dV, dK.  MODE_Q: S, dP (even tiles), dQ, dP (odd tiles).
  constexpr uint32_t S_COL = 0, DP_COL = 128, ACC0_COL = 256, ACC1_COL = 384;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) report_error(p.err, ERR_BOUNDS, 0xA7B1u);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* stat_full = bars;          // 1
  uint64_t* a_full = bars + 1;         // 3
  uint64_t* a_empty = bars + 4;        // 3
  uint64_t* b_full = bars + 7;         // 1
  uint64_t* b_empty = bars + 8;        // 1
  uint64_t* s_full = bars + 9;         // S of tile n is in TMEM
  uint64_t* dp_full = bars + 10;       // 2: dP of tile n is in TMEM (barrier n & 1)
  uint64_t* s_free = bars + 12;        // one arrival per element-wise warp: S of tile n has been read (MODE_KV: and P is in shared memory)
  uint64_t* pds_full = bars + 13;      // one arrival per element-wise warp: dS of tile n is in shared memory, dP has been read
  uint64_t* ds_free = bars + 14;       // MODE_Q: the dQ GEMM of tile n has finished reading dS
  uint64_t* acc_done = bars + 15;      // every GEMM of the current work item has completed
  uint64_t* stat_empty = bars + 16;    // the last S / dP GEMM of the work item has read the stationary tiles
  uint64_t* acc_free = bars + 17;
  uint64_t* p_ready = bars + 18;       // MODE_KV, one arrival per warp: P of tile n is in shared memory
  uint64_t* p_free = bars + 19;        // MODE_KV: the dV GEMM of tile n has finished reading P
  // acc_free: one arrival per warp: the accumulators of the work item have been read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q = (p.Sq + BLK - 1) / BLK;
  const int n_kv = (p.Sk + BLK - 1) / BLK;
  // Persistent CTAs: work item w = (owned tile, head, batch), tile-major so that under a causal mask
  // the long items come first; CTA c takes items c, c + gridDim.x, ...  Barrier phases run on over
  // the items (g counts streamed tiles, it counts items), so TMEM, the barriers and the pipelines
  // are set up once and the loads of the next item overlap the tail of the current one.
  const int hb = p.H * p.B;
  const int total_items = (MODE == MODE_KV ? n_kv : n_q) * hb;
  struct Item { int own, h, b, t_begin, n_iter; };
  auto item_at = [&](int w) {
    Item I;
    const int idx = w / hb, rem = w - idx * hb;
    I.own = MODE == MODE_KV ? idx : n_q - 1 - idx;
    I.h = rem % p.H;
    I.b = rem / p.H;
    I.t_begin = MODE == MODE_KV ? (p.causal ? I.own : 0) : 0;
    const int t_end = MODE == MODE_KV ? n_q : (p.causal ? min(I.own + 1, n_kv) : n_kv);
    I.n_iter = max(t_end - I.t_begin, 0);
    return I;
  };

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(stat_full), 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(smem_u32(&a_full[s]), 1);
      mbar_init(smem_u32(&a_empty[s]), 1);
    }
    mbar_init(smem_u32(b_full), 1);
    mbar_init(smem_u32(b_empty), 1);
    mbar_init(smem_u32(&dp_full[0]), 1);
    mbar_init(smem_u32(&dp_full[1]), 1);
    mbar_init(smem_u32(p_ready), EW_WARPS);
    mbar_init(smem_u32(p_free), 1);
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_free), EW_WARPS);        // one arrival per warp: 512 arrivals on one word cost ~0.5 us
    mbar_init(smem_u32(pds_full), EW_WARPS);
    mbar_init(smem_u32(ds_free), 1);
    mbar_init(smem_u32(acc_done), 1);
    mbar_init(smem_u32(stat_empty), 1);
    mbar_init(smem_u32(acc_free), EW_WARPS);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == EW_WARPS + 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == EW_WARPS) {
    // ---------------------------- TMA producer -----------------------------------------
    if (lane == 0) {
      const CUtensorMap* st0 = MODE == MODE_KV ? &tmK : &tmQ;
      const CUtensorMap* st1 = MODE == MODE_KV ? &tmV : &tmdO;
      const CUtensorMap* ma = MODE == MODE_KV ? &tmQ : &tmK;
      const CUtensorMap* mb = MODE == MODE_KV ? &tmdO : &tmV;
      int g = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        const Item I = item_at(w);
        if (I.n_iter == 0) continue;
        if (!(ok = mbar_wait(smem_u32(stat_empty), (it & 1) ^ 1u, abort_flag))) break;
        const uint32_t sb = smem_u32(stat_full);
        mbar_arrive_expect_tx(sb, 2 * L::TILE);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_4d(smem_u32(smem + L::STAT0_OFF + kb * (BLK * 128)), st0, sb, kb * 64, I.h, I.own * BLK, I.b);
          tma_load_4d(smem_u32(smem + L::STAT1_OFF + kb * (BLK * 128)), st1, sb, kb * 64, I.h, I.own * BLK, I.b);
        }
        for (int n = 0; n < I.n_iter && ok; ++n, ++g) {
          const int row0 = (I.t_begin + n) * BLK;
          {
            const int slot = g % NA;
            if (!(ok = mbar_wait(smem_u32(&a_empty[slot]), ((g / NA) & 1) ^ 1u, abort_flag))) break;
            const uint32_t fb = smem_u32(&a_full[slot]);
            mbar_arrive_expect_tx(fb, L::TILE);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem_u32(smem + L::A_OFF + slot * L::TILE + kb * (BLK * 128)), ma, fb, kb * 64, I.h, row0, I.b);
          }
          {
            const int slot = g % NB;
            if (!(ok = mbar_wait(smem_u32(&b_empty[slot]), ((g / NB) & 1) ^ 1u, abort_flag))) break;
            const uint32_t fb = smem_u32(&b_full[slot]);
            mbar_arrive_expect_tx(fb, L::TILE);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem_u32(smem + L::B_OFF + slot * L::TILE + kb * (BLK * 128)), mb, fb, kb * 64, I.h, row0, I.b);
          }
        }
        ++it;
      }
    }
  } else if (warp == EW_WARPS + 1) {
    // ---------------------------- MMA issuer -------------------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);   // S, dP
      constexpr uint32_t idesc_t = make_idesc_bf16(BLK, D, true, true);       // dV, dK
      constexpr uint32_t idesc_q = make_idesc_bf16(BLK, D, false, true);      // dQ
      constexpr uint32_t HI = smem_desc_hi(1024);
      // descriptor low words of every tile: K-major view (16-byte leading offset) and MN-major view
      // (64-column blocks BLK*128 bytes apart); a K step adds a constant
      const uint32_t st0_k = smem_desc_lo(smem_u32(smem + L::STAT0_OFF), 16);
      const uint32_t st1_k = smem_desc_lo(smem_u32(smem + L::STAT1_OFF), 16);
      const uint32_t ds_k = smem_desc_lo(smem_u32(smem + L::DS_OFF), 16);
      const uint32_t ds_mn = smem_desc_lo(smem_u32(smem + L::DS_OFF), BLK * 128);
      const uint32_t p_mn = smem_desc_lo(smem_u32(smem + L::P_OFF), BLK * 128);
      auto a_k = [&](int n) { return smem_desc_lo(smem_u32(smem + L::A_OFF + (n % NA) * L::TILE), 16); };
      auto a_mn = [&](int n) { return smem_desc_lo(smem_u32(smem + L::A_OFF + (n % NA) * L::TILE), BLK * 128); };
      auto b_k = [&](int n) { return smem_desc_lo(smem_u32(smem + L::B_OFF + (n % NB) * L::TILE), 16); };
      auto b_mn = [&](int n) { return smem_desc_lo(smem_u32(smem + L::B_OFF + (n % NB) * L::TILE), BLK * 128); };
      auto wait_a = [&](int n) { return mbar_wait(smem_u32(&a_full[n % NA]), (n / NA) & 1, abort_flag); };
      auto wait_b = [&](int n) { return mbar_wait(smem_u32(&b_full[n % NB]), (n / NB) & 1, abort_flag); };
      // S = Q·Kᵀ and dP = dO·Vᵀ: both operands K-major, D/16 K steps
      auto issue_sdp = [&](uint32_t col, uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t off = (kb * (BLK * 128) + k * 32) >> 4;
            umma_bf16_ss_split(tmem_base + col, a_lo + off, HI, b_lo + off, HI, idesc_s, (kb | k) != 0 ? 1u : 0u);
          }
      };
      // accumulate GEMMs over the 128 rows of the streamed tile: A and B read through MN-major views
      auto issue_acc_mn = [&](uint32_t col, uint32_t a_lo, uint32_t b_lo, bool acc_first) {
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {
          const uint32_t off = (kk * (16 * 128)) >> 4;
          umma_bf16_ss_split(tmem_base + col, a_lo + off, HI, b_lo + off, HI, idesc_t, (acc_first || kk != 0) ? 1u : 0u);
        }
      };
      auto issue_s = [&](int n) {
        if (MODE == MODE_KV) issue_sdp(S_COL, a_k(n), st0_k); else issue_sdp(S_COL, st0_k, a_k(n));
        umma_commit(smem_u32(s_full));
      };
      auto issue_dp = [&](int n) {
        const uint32_t col = (MODE == MODE_Q && (n & 1)) ? ACC1_COL : DP_COL;
        if (MODE == MODE_KV) issue_sdp(col, b_k(n), st1_k); else issue_sdp(col, st1_k, b_k(n));
        umma_commit(smem_u32(&dp_full[n & 1]));
        if (MODE == MODE_Q) umma_commit(smem_u32(&b_empty[n % NB]));   // V is only needed by dP
      };
      int g = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        const Item I = item_at(w);
        if (I.n_iter == 0) continue;
        // prologue: S and dP of the item's first tile.  Their TMEM columns are free: every iteration,
        // the previous item's last one included, waits for s_free and pds_full.
        if (!(ok = mbar_wait(smem_u32(stat_full), it & 1, abort_flag))) break;
        if (!(ok = wait_a(g))) break;
        tc_fence_after();
        issue_s(g);
        if (!(ok = wait_b(g))) break;
        tc_fence_after();
        issue_dp(g);
        for (int n = 0; n < I.n_iter && ok; ++n, ++g) {
          const bool more = n + 1 < I.n_iter;
          // every S / dP GEMM of the item has been issued: the stationary tiles can be replaced
          // as soon as those complete
          if (!more) umma_commit(smem_u32(stat_empty));
          if (!(ok = mbar_wait(smem_u32(s_free), g & 1, abort_flag))) break;
          // the first accumulate GEMM of an item overwrites accumulators that the element-wise warps
          // may still be reading out for the previous item
          if (n == 0 && it > 0 && !(ok = mbar_wait(smem_u32(acc_free), (it - 1) & 1, abort_flag))) break;
          tc_fence_after();
          if (more) {
            // S of the next tile, as soon as this tile's S has been read
            if (!(ok = wait_a(g + 1))) break;
            tc_fence_after();
            issue_s(g + 1);
            if (MODE == MODE_Q) {
              // dP of the next tile goes to the other dP buffer, read last by tile g-1
              if (!(ok = wait_b(g + 1))) break;
              tc_fence_after();
              issue_dp(g + 1);
            }
          }
          if (MODE == MODE_KV) {
            // dV[kv, d] += sum_q P[q, kv] dO[q, d], once P has been stored (S of the next tile is already
            // running: the element-wise warps release S before they convert and store P)
            if (!(ok = mbar_wait(smem_u32(p_ready), g & 1, abort_flag))) break;
            tc_fence_after();
            issue_acc_mn(ACC0_COL, p_mn, b_mn(g), n != 0);
            umma_commit(smem_u32(&b_empty[g % NB]));
            umma_commit(smem_u32(p_free));
          }
          if (!(ok = mbar_wait(smem_u32(pds_full), g & 1, abort_flag))) break;
          tc_fence_after();
          if (MODE == MODE_KV) {
            // dK[kv, d] += sum_q dS[q, kv] Q[q, d]
            issue_acc_mn(ACC1_COL, ds_mn, a_mn(g), n != 0);
            umma_commit(smem_u32(&a_empty[g % NA]));
          } else {
            // dQ[q, d] += sum_kv dS[q, kv] K[kv, d]: dS K-major, K through its MN-major view
            const uint32_t k_lo = a_mn(g);
#pragma unroll
            for (int kk = 0; kk < BLK / 16; ++kk)
              umma_bf16_ss_split(tmem_base + ACC0_COL, ds_k + (((kk >> 2) * (BLK * 128) + (kk & 3) * 32) >> 4), HI,
                                 k_lo + ((kk * (16 * 128)) >> 4), HI, idesc_q, (n | kk) != 0 ? 1u : 0u);
            umma_commit(smem_u32(&a_empty[g % NA]));
            umma_commit(smem_u32(ds_free));
          }
          if (!more) {
            umma_commit(smem_u32(acc_done));
          } else if (MODE == MODE_KV) {
            // dP of the next tile: its columns were read before pds_full(g) completed
            if (!(ok = wait_b(g + 1))) break;
            tc_fence_after();
            issue_dp(g + 1);
          }
        }
        ++it;
      }
    }
  } else {
    // ---------------------------- element-wise warps -----------------------------------
    const int quad = warp & 3;
    const int part = warp >> 2;                 // which 32 key columns of the tile this thread handles
    const int r = quad * 32 + lane;             // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    int g = 0, it = 0;
    for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
    const Item I = item_at(w);
    const int own = I.own, h = I.h, b = I.b, t_begin = I.t_begin, n_iter = I.n_iter;
    float lse2 = 0.0f, dlt = 0.0f;
    int row_g = own * BLK + r;
    bool row_ok = row_g < p.Sq;
    if (MODE == MODE_Q && row_ok) {
      const long long stat_idx = ((long long)b * p.H + h) * p.Sq + row_g;
      lse2 = p.lse[stat_idx] * LOG2E;
      dlt = p.delta[stat_idx];
    }
    float lse_next = 0.0f, dlt_next = 0.0f;      // MODE_KV: statistics of the next query tile's row
    if (MODE == MODE_KV && n_iter > 0 && t_begin * BLK + r < p.Sq) {
      const long long stat_idx = ((long long)b * p.H + h) * p.Sq + t_begin * BLK + r;
      lse_next = p.lse[stat_idx];
      dlt_next = p.delta[stat_idx];
    }
    for (int n = 0; n < n_iter; ++n, ++g) {
      const int t = t_begin + n;                               // streamed tile index
      const int q_tile = MODE == MODE_KV ? t : own;
      const int kv_tile = MODE == MODE_KV ? own : t;
      if (MODE == MODE_KV) {
        // this tile's row statistics were loaded one iteration ago; start the loads for the next tile
        // now so that their latency hides behind this iteration
        row_g = q_tile * BLK + r;
        row_ok = row_g < p.Sq;
        lse2 = lse_next * LOG2E;
        dlt = dlt_next;
        const int row_n = row_g + BLK;
        if (n + 1 < n_iter && row_n < p.Sq) {
          const long long stat_idx = ((long long)b * p.H + h) * p.Sq + row_n;
          lse_next = p.lse[stat_idx];
          dlt_next = p.delta[stat_idx];
        } else {
          lse_next = 0.0f;
          dlt_next = 0.0f;
        }
      }
      const int kv0 = kv_tile * BLK;
      // tiles that need no masking: every row and column valid and strictly below the diagonal
      constexpr bool biased = BIAS;   // additive biases / valid lengths: a separate instantiation, the plain one is unchanged
      const bool plain = (q_tile + 1) * BLK <= p.Sq && (kv_tile + 1) * BLK <= p.Sk &&
                         !(p.causal && kv_tile >= q_tile) && !biased;
      float pv[32];
      uint8_t* const p_tile = smem + L::P_OFF + (part >> 1) * (BLK * 128);    // 64-column block of the P / dS tile
      uint8_t* const ds_tile = smem + L::DS_OFF + (part >> 1) * (BLK * 128);
      const int c16_0 = (part & 1) * 4;                                        // first 16-byte chunk inside the 128-byte row
      // ---- phase A: P = exp2(S·c − lse) --------------------------------------------------
      // s_full(n) was committed after the dV GEMM of tile n-1: the P buffer is free
      if (!mbar_wait_warp(smem_u32(s_full), g & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t s_r[32];
        tmem_ld_32x32(tmem_base + lane_off + S_COL + part * 32, s_r);
        tmem_ld_wait();
        if (plain) {
#pragma unroll
          for (int q = 0; q < 32; ++q) pv[q] = fast_exp2(__uint_as_float(s_r[q]) * p.scale_log2 - lse2);
        } else if constexpr (!biased) {
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            const int colg = kv0 + part * 32 + q;
            const bool dead = !row_ok || colg >= p.Sk || (p.causal && colg > row_g);
            pv[q] = dead ? 0.0f : fast_exp2(__uint_as_float(s_r[q]) * p.scale_log2 - lse2);
          }
        } else {
          // the forward's logits were scale * q·k + key_bias + attn_bias with keys (and queries) beyond the
          // valid length masked; a fully masked row has lse = -inf and contributes nothing
          int kv_len = p.Sk;
          if (p.lengths) kv_len = max(0, min(p.Sk, p.lengths[b]));
          const bool row_live = row_ok && (!p.lengths || row_g < kv_len) && lse2 > -INFINITY;
          const float* kb = p.key_bias ? p.key_bias + (long long)b * p.kb_sb + (long long)h * p.kb_sh : nullptr;
          const float* ab = (p.attn_bias && row_ok)
                                ? p.attn_bias + (long long)b * p.ab_sb + (long long)h * p.ab_sh + (long long)row_g * p.ab_sq
                                : nullptr;
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            const int colg = kv0 + part * 32 + q;
            const bool dead = !row_live || colg >= kv_len || (p.causal && colg > row_g);
            float e = 0.0f;
            if (!dead) {
              float bias = kb ? kb[colg] : 0.0f;
              if (ab) bias += ab[colg];
              e = fast_exp2(fmaf(__uint_as_float(s_r[q]), p.scale_log2, bias * LOG2E) - lse2);
            }
            pv[q] = e;
          }
        }
      }
      // S has been read: the next S GEMM may overwrite it while P is converted and stored
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(s_free));
      if (MODE == MODE_KV) {
        // the dV GEMM of the previous tile must have finished reading the P buffer
        if (g > 0 && !mbar_wait_warp(smem_u32(p_free), (g - 1) & 1, abort_flag)) { ok = false; break; }
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) store8_bf16(p_tile, r, c16_0 + c8, &pv[c8 * 8]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(p_ready));
      }
      // ---- phase B: dS = P∘(dP − delta) → shared memory ---------------------------------------
      if (!mbar_wait_warp(smem_u32(&dp_full[g & 1]), (g >> 1) & 1, abort_flag)) { ok = false; break; }
      // the previous tile's GEMM that reads the dS buffer must be done: in the dK/dV pass dP(n) was
      // issued after it; the dQ pass issues dP early and signals the buffer separately
      if (MODE == MODE_Q && g > 0 && !mbar_wait_warp(smem_u32(ds_free), (g - 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t dp_col = (MODE == MODE_Q && (g & 1)) ? ACC1_COL : DP_COL;
      {
        uint32_t dp_r[32];
        tmem_ld_32x32(tmem_base + lane_off + dp_col + part * 32, dp_r);
        tmem_ld_wait();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float dsv[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) dsv[q] = pv[c8 * 8 + q] * (__uint_as_float(dp_r[c8 * 8 + q]) - dlt);
          store8_bf16(ds_tile, r, c16_0 + c8, dsv);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(pds_full));
    }
    if (ok && n_iter > 0 && !mbar_wait_warp(smem_u32(acc_done), it & 1, abort_flag)) ok = false;
    if (ok && n_iter > 0) {
      tc_fence_after();
      // 32 accumulator columns per thread: chunk `part` (and, for D > 128, every fourth one after it)
      const int own_row = own * BLK + r;
      for (int ch = part; ch < D / 32; ch += EW_WARPS / 4) {
        if (MODE == MODE_KV) {
          const bool kv_ok = own_row < p.Sk;
          __nv_bfloat16* dvp = p.dV + (long long)b * p.dv_sb + (long long)own_row * p.dv_ss + (long long)h * p.dv_sh + ch * 32;
          __nv_bfloat16* dkp = p.dK + (long long)b * p.dk_sb + (long long)own_row * p.dk_ss + (long long)h * p.dk_sh + ch * 32;
          // TMEM loads are warp-collective: every lane issues them, only the stores are predicated
          uint32_t tv[32], tk[32];
          tmem_ld_32x32(tmem_base + lane_off + ACC0_COL + ch * 32, tv);
          tmem_ld_32x32(tmem_base + lane_off + ACC1_COL + ch * 32, tk);
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
              reinterpret_cast<uint4*>(dvp)[q] = uv;
              reinterpret_cast<uint4*>(dkp)[q] = uk;
            }
          }
        } else {
          const bool q_ok = own_row < p.Sq;
          __nv_bfloat16* dqp = p.dQ + (long long)b * p.dq_sb + (long long)own_row * p.dq_ss + (long long)h * p.dq_sh + ch * 32;
          uint32_t tq[32];
          tmem_ld_32x32(tmem_base + lane_off + ACC0_COL + ch * 32, tq);
          tmem_ld_wait();
          if (q_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(tq[q * 8 + 0]) * p.scale, __uint_as_float(tq[q * 8 + 1]) * p.scale);
              u.y = pack_bf16x2(__uint_as_float(tq[q * 8 + 2]) * p.scale, __uint_as_float(tq[q * 8 + 3]) * p.scale);
              u.z = pack_bf16x2(__uint_as_float(tq[q * 8 + 4]) * p.scale, __uint_as_float(tq[q * 8 + 5]) * p.scale);
              u.w = pack_bf16x2(__uint_as_float(tq[q * 8 + 6]) * p.scale, __uint_as_float(tq[q * 8 + 7]) * p.scale);
              reinterpret_cast<uint4*>(dqp)[q] = u;
            }
          }
        }
      }
    }
    if (ok && n_iter > 0) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_free));
      ++it;
    }
    if (n_iter == 0 && part == 0) {
      // nothing attends to / from this tile: its gradient rows are zero
      const uint4 z = make_uint4(0, 0, 0, 0);
      const int own_row = own * BLK + r;
      if (MODE == MODE_KV) {
        if (own_row < p.Sk) {
          __nv_bfloat16* dvp = p.dV + (long long)b * p.dv_sb + (long long)own_row * p.dv_ss + (long long)h * p.dv_sh;
          __nv_bfloat16* dkp = p.dK + (long long)b * p.dk_sb + (long long)own_row * p.dk_ss + (long long)h * p.dk_sh;
          for (int q = 0; q < D / 8; ++q) {
            reinterpret_cast<uint4*>(dvp)[q] = z;
            reinterpret_cast<uint4*>(dkp)[q] = z;
          }
        }
      } else if (own_row < p.Sq) {
        __nv_bfloat16* dqp = p.dQ + (long long)b * p.dq_sb + (long long)own_row * p.dq_ss + (long long)h * p.dq_sh;
        for (int q = 0; q < D / 8; ++q) reinterpret_cast<uint4*>(dqp)[q] = z;
      }
    }
    }   // work items
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_error(p.err, ERR_MBAR_TIMEOUT, 0xA7B0u + MODE);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == EW_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d].  D / 8 lanes share one (b,s,h) row, each with one
// 16-byte load of O and of dO (a warp covers 2 rows at D = 128, 4 at D = 64): one row per warp with 4-byte
// loads left this bandwidth-bound pass at a quarter of the copy rate.
template <int D>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                  float* __restrict__ delta, int B, int S, int H, long long o_sb, long long o_ss, long long o_sh,
                  long long do_sb, long long do_ss, long long do_sh) {
  constexpr int LPR = D / 8;                       // lanes per row
  const long long total = (long long)B * S * H;
  const int sub = threadIdx.x % LPR;
  const long long stride = (long long)gridDim.x * (blockDim.x / LPR);
  for (long long w = blockIdx.x * (long long)(blockDim.x / LPR) + threadIdx.x / LPR; ; w += stride) {
    // every lane of a warp takes the same number of trips: the shuffles below need the full warp
    const bool live = w < total;
    if (!__any_sync(0xffffffffu, live)) break;
    float acc = 0.0f;
    int hh = 0, s = 0, bb = 0;
    if (live) {
      hh = (int)(w % H);
      const long long bs = w / H;
      s = (int)(bs % S);
      bb = (int)(bs / S);
      const uint4 a = *reinterpret_cast<const uint4*>(O + bb * o_sb + s * o_ss + hh * o_sh + sub * 8);
      const uint4 g = *reinterpret_cast<const uint4*>(dO + bb * do_sb + s * do_ss + hh * do_sh + sub * 8);
      const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack_bf16x2(av[i]), y = unpack_bf16x2(gv[i]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (live && sub == 0) delta[((long long)bb * H + hh) * S + s] = acc;
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
  // optional additive biases (fp32) and valid lengths (int32 [B]) of the forward pass; null = absent
  const float* key_bias;  long long kb_sb, kb_sh;
  const float* attn_bias; long long ab_sb, ab_sh, ab_sq;
  const int* lengths;
};

// delta: fp32 [B,H,Sq] workspace.  dQ_acc is unused (kept in the argument block for ABI stability).
ST_API int st_attn_bwd(const StAttnBwdArgs* a, void* stream_v) {
  if (!a || !a->Q || !a->K || !a->V || !a->O || !a->dO || !a->lse || !a->delta ||
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
  const void* ptrs[] = {a->Q, a->K, a->V, a->O, a->dO, a->dQ, a->dK, a->dV};
  for (const void* q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) & 15) return st::fail(ST_ERR_INVALID, "attn_bwd: pointers must be 16-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);

  {
    const long long rows = (long long)a->B * a->Sq * a->H;
    const int rows_per_block = 256 / (a->D / 8);
    long long blocks = (rows + rows_per_block - 1) / rows_per_block;
    if (blocks > 148 * 16) blocks = 148 * 16;
    auto Op = static_cast<const __nv_bfloat16*>(a->O);
    auto dOp = static_cast<const __nv_bfloat16*>(a->dO);
    if (a->D == 128)
      attn_delta_kernel<128><<<(unsigned)blocks, 256, 0, s>>>(Op, dOp, a->delta, a->B, a->Sq, a->H, a->o_sb, a->o_ss,
                                                            a->o_sh, a->do_sb, a->do_ss, a->do_sh);
    else
      attn_delta_kernel<64><<<(unsigned)blocks, 256, 0, s>>>(Op, dOp, a->delta, a->B, a->Sq, a->H, a->o_sb, a->o_ss,
                                                           a->o_sh, a->do_sb, a->do_ss, a->do_sh);
    ST_CUDA_CHECK(cudaGetLastError());
  }

  CUtensorMap tq, tk, tv, tdo;
  if (!st::encode_bshd_tmap(&tq, a->Q, a->B, a->Sq, a->H, a->D, a->q_sb, a->q_ss, a->q_sh, BLK) ||
      !st::encode_bshd_tmap(&tk, a->K, a->B, a->Sk, a->H, a->D, a->k_sb, a->k_ss, a->k_sh, BLK) ||
      !st::encode_bshd_tmap(&tv, a->V, a->B, a->Sk, a->H, a->D, a->v_sb, a->v_ss, a->v_sh, BLK) ||
      !st::encode_bshd_tmap(&tdo, a->dO, a->B, a->Sq, a->H, a->D, a->do_sb, a->do_ss, a->do_sh, BLK))
    return ST_ERR_CUDA;
  AttnBwdParams p;
  p.lse = a->lse; p.delta = a->delta;
  p.dQ = static_cast<__nv_bfloat16*>(a->dQ);
  p.dK = static_cast<__nv_bfloat16*>(a->dK);
  p.dV = static_cast<__nv_bfloat16*>(a->dV);
  p.dq_sb = a->dq_sb; p.dq_ss = a->dq_ss; p.dq_sh = a->dq_sh;
  p.dk_sb = a->dk_sb; p.dk_ss = a->dk_ss; p.dk_sh = a->dk_sh;
  p.dv_sb = a->dv_sb; p.dv_ss = a->dv_ss; p.dv_sh = a->dv_sh;
  p.B = a->B; p.H = a->H; p.Sq = a->Sq; p.Sk = a->Sk;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.causal = a->causal;
  p.err = st::error_word();
  p.key_bias = a->key_bias; p.kb_sb = a->kb_sb; p.kb_sh = a->kb_sh;
  p.attn_bias = a->attn_bias; p.ab_sb = a->ab_sb; p.ab_sh = a->ab_sh; p.ab_sq = a->ab_sq;
  p.lengths = a->lengths;
  const bool biased = a->key_bias || a->attn_bias || a->lengths;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    ST_CUDA_CHECK(cudaGetDevice(&dev));
    ST_CUDA_CHECK(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const int items_kv = ((a->Sk + BLK - 1) / BLK) * a->H * a->B;
  const int items_q = ((a->Sq + BLK - 1) / BLK) * a->H * a->B;
  const dim3 grid_kv(items_kv < num_sms ? items_kv : num_sms);
  const dim3 grid_q(items_q < num_sms ? items_q : num_sms);
  auto launch = [&](auto kernel, int smem_bytes, dim3 grid) -> int {
    ST_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    kernel<<<grid, NUM_THREADS, smem_bytes, s>>>(tq, tk, tv, tdo, p);
    ST_CUDA_CHECK(cudaGetLastError());
    return ST_OK;
  };
  int rc;
  if (a->D == 128) {
    if (biased) {
      if ((rc = launch(attn_bwd_kernel<128, MODE_KV, true>, BwdSmem<128, MODE_KV>::TOTAL, grid_kv)) != ST_OK) return rc;
      if ((rc = launch(attn_bwd_kernel<128, MODE_Q, true>, BwdSmem<128, MODE_Q>::TOTAL, grid_q)) != ST_OK) return rc;
    } else {
      if ((rc = launch(attn_bwd_kernel<128, MODE_KV, false>, BwdSmem<128, MODE_KV>::TOTAL, grid_kv)) != ST_OK) return rc;
      if ((rc = launch(attn_bwd_kernel<128, MODE_Q, false>, BwdSmem<128, MODE_Q>::TOTAL, grid_q)) != ST_OK) return rc;
    }
  } else {
    if (biased) {
      if ((rc = launch(attn_bwd_kernel<64, MODE_KV, true>, BwdSmem<64, MODE_KV>::TOTAL, grid_kv)) != ST_OK) return rc;
      if ((rc = launch(attn_bwd_kernel<64, MODE_Q, true>, BwdSmem<64, MODE_Q>::TOTAL, grid_q)) != ST_OK) return rc;
    } else {
      if ((rc = launch(attn_bwd_kernel<64, MODE_KV, false>, BwdSmem<64, MODE_KV>::TOTAL, grid_kv)) != ST_OK) return rc;
      if ((rc = launch(attn_bwd_kernel<64, MODE_Q, false>, BwdSmem<64, MODE_Q>::TOTAL, grid_q)) != ST_OK) return rc;
    }
  }
  return ST_OK;
}
