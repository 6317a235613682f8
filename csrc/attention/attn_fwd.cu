// Attention forward with online softmax on sm_100a tensor cores.
//
// One CTA owns a 128-row query tile of one (batch, head).  Per 128-row KV tile:
//   S  = Q·Kᵀ            tcgen05.mma, fp32 in TMEM (two S buffers)
//   P  = exp2(S·c − m)   eight softmax warps, two threads per row (64 columns each); the
//                        running max is exchanged through shared memory, P goes to shared
//                        memory as bf16 in the 128-byte-swizzled K-major layout
//   PV = P·V             tcgen05.mma into a fresh TMEM buffer (two PV buffers)
//   O  = O·α + PV        in registers, deferred by one tile so that it overlaps the next
//                        QKᵀ and softmax
// Warp 8 is the TMA producer (double-buffered K and V), warp 9 issues the MMAs and owns
// TMEM.  Causal masking assumes seq_q == seq_k; KV tiles above the diagonal are skipped and
// heavy query tiles are scheduled first.
//
// Outputs O (bf16, [B,S,H,D] strided) and the log-sum-exp per row (fp32 [B,H,S]).
//
// The BIAS instantiation adds, before the softmax, a per-key bias key_bias[b, (h,) key] and / or a
// per-(query, key) bias attn_bias[b, (h,) query, key] (both fp32, added to scale * q·k), and honours a
// valid length per batch entry: keys at or beyond lengths[b] are masked and queries at or beyond it
// produce zeros (the semantics of the reference's z_bias / attn_bias / context_lengths arguments,
// crates/st-core/src/backend/cuda_attention.cu:85-96,117-202).  The plain instantiation is unchanged.
//
// Reference parity: fused_attention_online.wgsl (crates/st-backend-wgpu/src/shaders),
// scaled_dot_attention_kernel (crates/st-core/src/backend/cuda_attention.cu:80-258),
// fused_attention_cpu (crates/st-tensor/src/pure.rs:11845-11919).
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {
using namespace st;

constexpr int BLK = 128;           // query rows and KV rows per tile
constexpr int NUM_THREADS = 320;   // 8 softmax warps + producer + MMA

struct AttnFwdParams {
  __nv_bfloat16* O;
  float* lse;
  long long o_sb, o_ss, o_sh;  // element strides of O for batch, sequence, head
  int B, H, Sq, Sk;
  float scale_log2;            // softmax scale * log2(e)
  int causal;
  unsigned* err;
  int n_q;       // query tiles per (batch, head)
  int n_items;   // n_q * H * B work items, heaviest (latest) query tiles first
  // ---- BIAS instantiation only ----
  const float* key_bias;       // [B, (H,) Sk] or null; element strides kb_sb, kb_sh (0 = shared by the heads)
  const float* attn_bias;      // [B, (H,) Sq, Sk] or null; element strides ab_sb, ab_sh, ab_sq (keys contiguous)
  const int* lengths;          // [B] valid keys (and queries) per batch entry, or null
  long long kb_sb, kb_sh, ab_sb, ab_sh, ab_sq;
  // ---- pair kernel only: optional phase clock sums of CTA 0 (null = off) ----
  unsigned long long* trace;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void pair_sync(int quad) {
  asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");
}

template <int D>
struct FwdSmem {
  static constexpr int TILE = BLK * D * 2;       // bytes of a Q / K / V tile
  static constexpr int P_TILE = BLK * BLK * 2;   // bytes of a P tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILE;
  static constexpr int V_OFF = K_OFF + 2 * TILE;
  static constexpr int P_OFF = V_OFF + 2 * TILE;
  static constexpr int BAR_OFF = P_OFF + 2 * P_TILE;
  static constexpr int XCH_OFF = BAR_OFF + 256;           // 2 x 2 x 128 floats (max exchange)
  static constexpr int TOTAL = XCH_OFF + 2 * 2 * BLK * 4;
};

template <int D, bool BIAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using L = FwdSmem<D>;
  constexpr int DH = D / 2;            // output columns per softmax thread
  constexpr int KB = D / 64;           // 64-wide (128-byte) blocks along D
  constexpr uint32_t S_COL = 0, PV_COL = 256;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned base (uniform exit)
    if (threadIdx.x == 0) report_error(p.err, ERR_BOUNDS, 0xA7F1u);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* v_full = bars + 3;      // 2
  uint64_t* k_empty = bars + 5;     // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* p_full = bars + 11;     // 2 (256 arrivals)
  uint64_t* pv_full = bars + 13;    // 2
  uint64_t* q_empty = bars + 15;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(smem + L::XCH_OFF);  // [2 buffers][2 halves][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work item w -> (query tile, head, batch); tiles with the most KV work come first so that the
  // static round-robin over CTAs stays balanced.
  const int hb = p.H * p.B;
  auto item_at = [&](int w, int& q_tile, int& h, int& b, int& n_kv) {
    q_tile = p.n_q - 1 - w / hb;
    const int rem = w % hb;
    h = rem % p.H;
    b = rem / p.H;
    int kv_len = p.Sk;
    if (BIAS && p.lengths) kv_len = max(0, min(p.Sk, p.lengths[b]));
    n_kv = (kv_len + BLK - 1) / BLK;
    if (p.causal) n_kv = min(n_kv, q_tile + 1);
    if (BIAS && p.lengths && q_tile * BLK >= kv_len) n_kv = 0;   // every query of the tile is beyond the valid length
  };

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    mbar_init(smem_u32(q_empty), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&k_full[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1);
      mbar_init(smem_u32(&k_empty[i]), 1);
      mbar_init(smem_u32(&v_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&p_full[i]), 8);     // one arrival per softmax warp
      mbar_init(smem_u32(&pv_full[i]), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
    if (lane == 0) {
      int g = 0;  // KV tiles loaded so far, over all work items: ring stage g & 1
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
        int q_tile, h, b, n_kv;
        item_at(w, q_tile, h, b, n_kv);
        if (n_kv <= 0) continue;
        // the single Q buffer is free once the previous item's last QK^T has completed
        if (it > 0 && !mbar_wait(smem_u32(q_empty), (it - 1) & 1, abort_flag)) break;
        const uint32_t qb = smem_u32(q_full);
        mbar_arrive_expect_tx(qb, L::TILE);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(smem_u32(smem + L::Q_OFF + kb * (BLK * 128)), &tmQ, qb, kb * 64, h, q_tile * BLK, b);
        for (int j = 0; j < n_kv; ++j, ++g) {
          const int st = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          if (!mbar_wait(smem_u32(&k_empty[st]), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t kf = smem_u32(&k_full[st]);
          mbar_arrive_expect_tx(kf, L::TILE);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_4d(smem_u32(smem + L::K_OFF + st * L::TILE + kb * (BLK * 128)), &tmK, kf,
                        kb * 64, h, j * BLK, b);
          if (!mbar_wait(smem_u32(&v_empty[st]), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t vf = smem_u32(&v_full[st]);
          mbar_arrive_expect_tx(vf, L::TILE);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_4d(smem_u32(smem + L::V_OFF + st * L::TILE + kb * (BLK * 128)), &tmV, vf,
                        kb * 64, h, j * BLK, b);
        }
        ++it;
      }
    }
  } else if (warp == 9) {
    // ---------------------------- MMA issuer -------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BLK, D, false, true);
      const uint32_t sq = smem_u32(smem + L::Q_OFF);
      // gg: KV tile index over all work items (ring stage, S / PV buffer and barrier phase)
      auto issue_qk = [&](int gg, bool last_of_item) -> bool {
        const int st = gg & 1;
        if (!mbar_wait(smem_u32(&k_full[st]), (gg >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::K_OFF + st * L::TILE);
        const uint32_t d_tmem = tmem_base + S_COL + st * BLK;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc_sw128(sq + kb * (BLK * 128) + k * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sk + kb * (BLK * 128) + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc_s, (kb | k) != 0 ? 1u : 0u);
          }
        umma_commit(smem_u32(&s_full[st]));
        umma_commit(smem_u32(&k_empty[st]));
        if (last_of_item) umma_commit(smem_u32(q_empty));
        return true;
      };
      int g = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
        int q_tile, h, b, n_kv;
        item_at(w, q_tile, h, b, n_kv);
        if (n_kv <= 0) continue;
        ok = mbar_wait(smem_u32(q_full), it & 1, abort_flag);
        if (ok) ok = issue_qk(g, n_kv == 1);
        for (int j = 0; j < n_kv && ok; ++j, ++g) {
          if (j + 1 < n_kv) {
            ok = issue_qk(g + 1, j + 2 == n_kv);
            if (!ok) break;
          }
          const int st = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          if (!mbar_wait(smem_u32(&p_full[st]), ph, abort_flag)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&v_full[st]), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sp = smem_u32(smem + L::P_OFF + st * L::P_TILE);
          const uint32_t sv = smem_u32(smem + L::V_OFF + st * L::TILE);
          const uint32_t d_tmem = tmem_base + PV_COL + st * D;
#pragma unroll
          for (int kk = 0; kk < BLK / 16; ++kk) {
            // A = P (K-major, two 64-column blocks); B = V (MN-major: D contiguous, KV rows = K)
            const uint64_t da = make_smem_desc_sw128(sp + (kk >> 2) * (BLK * 128) + (kk & 3) * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sv + kk * (16 * 128), BLK * 128, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc_pv, kk != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&pv_full[st]));
          umma_commit(smem_u32(&v_empty[st]));
        }
        ++it;
      }
    }
  } else {
    // ---------------------------- softmax / output warps -------------------------------
    const int quad = warp & 3;
    const int half = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float2 o[DH / 2];
    bool ok = true;
    int g0 = 0;  // KV tiles consumed by earlier work items (S / P / PV buffer index and barrier phase)

    auto accumulate = [&](int jj, float a) -> bool {
      const int pb = jj & 1;
      if (!mbar_wait_warp(smem_u32(&pv_full[pb]), (jj >> 1) & 1, abort_flag)) return false;
      tc_fence_after();
#pragma unroll
      for (int ch = 0; ch < DH / 32; ++ch) {
        uint32_t t[32];
        tmem_ld_32x32(tmem_base + lane_off + PV_COL + pb * D + half * DH + ch * 32, t);
        tmem_ld_wait();
        const float2 a2 = make_float2(a, a);
#pragma unroll
        for (int c = 0; c < 16; ++c)
          o[ch * 16 + c] = fma2(o[ch * 16 + c], a2,
                                make_float2(__uint_as_float(t[2 * c]), __uint_as_float(t[2 * c + 1])));
      }
      return true;
    };

    for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
    int q_tile, h, b, n_kv;
    item_at(w, q_tile, h, b, n_kv);
    const int q0 = q_tile * BLK;
    const int row_g = q0 + r;
    float m = -INFINITY, l = 0.0f, alpha_prev = 1.0f;
#pragma unroll
    for (int c = 0; c < DH / 2; ++c) o[c] = make_float2(0.0f, 0.0f);
    // BIAS: logits are moved to the log2 domain (scale and biases applied) before the maximum, so the
    // factor used afterwards is 1
    const float sc = BIAS ? 1.0f : p.scale_log2;
    int kv_len = p.Sk;
    if (BIAS && p.lengths) kv_len = max(0, min(p.Sk, p.lengths[b]));
    const bool row_live = !BIAS || row_g < kv_len || !p.lengths;

    for (int j = 0; j < n_kv; ++j) {
      const int gj = g0 + j;
      const int buf = gj & 1;
      if (!mbar_wait_warp(smem_u32(&s_full[buf]), (gj >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[64];
      {
        uint32_t t0[32], t1[32];
        const uint32_t ta = tmem_base + lane_off + S_COL + buf * BLK + half * 64;
        tmem_ld_32x32(ta, t0);
        tmem_ld_32x32(ta + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) { sr[c] = t0[c]; sr[32 + c] = t1[c]; }
      }
      const int col0 = j * BLK + half * 64;
      const bool need_mask = (p.causal && (j == q_tile)) || (col0 + 64 > p.Sk);
      float mx = -INFINITY;
      if constexpr (BIAS) {
        constexpr float LOG2E = 1.4426950408889634f;
        const float* kb = p.key_bias ? p.key_bias + (long long)b * p.kb_sb + (long long)h * p.kb_sh : nullptr;
        const float* ab = (p.attn_bias && row_g < p.Sq)
                              ? p.attn_bias + (long long)b * p.ab_sb + (long long)h * p.ab_sh + (long long)row_g * p.ab_sq
                              : nullptr;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int col = col0 + c;
          const bool dead = !row_live || col >= kv_len || (p.causal && col > row_g);
          float s = -INFINITY;
          if (!dead) {
            float bias = kb ? kb[col] : 0.0f;
            if (ab) bias += ab[col];
            s = fmaf(__uint_as_float(sr[c]), p.scale_log2, bias * LOG2E);
          }
          sr[c] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      } else if (need_mask) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int col = col0 + c;
          const bool dead = (col >= p.Sk) || (p.causal && col > row_g);
          float s = dead ? -INFINITY : __uint_as_float(sr[c]);
          sr[c] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      } else {
        float mx1 = -INFINITY;   // two chains of three-input maxima
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          mx = max3(mx, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
          mx1 = max3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
        }
        mx = fmaxf(mx, mx1);
      }
      float* xb = xch + buf * (2 * BLK);
      xb[half * BLK + r] = mx;
      pair_sync(quad);
      mx = fmaxf(mx, xb[(half ^ 1) * BLK + r]);
      const float m_new = fmaxf(m, mx * sc);
      const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = fast_exp2(m - m_safe);
      uint8_t* pt = smem + L::P_OFF + buf * L::P_TILE + half * (BLK * 128);
      const float2 sc2 = make_float2(sc, sc);
      const float2 nm2 = make_float2(-m_safe, -m_safe);
      float2 rs2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        float2 e[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 x = fma2(make_float2(__uint_as_float(sr[c8 * 8 + 2 * q]),
                                            __uint_as_float(sr[c8 * 8 + 2 * q + 1])), sc2, nm2);
          e[q] = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          rs2[q & 1] = add2(rs2[q & 1], e[q]);
        }
        uint4 u;
        u.x = pack_bf16x2(e[0].x, e[0].y); u.y = pack_bf16x2(e[1].x, e[1].y);
        u.z = pack_bf16x2(e[2].x, e[2].y); u.w = pack_bf16x2(e[3].x, e[3].y);
        *reinterpret_cast<uint4*>(pt + sw128_offset(r, c8)) = u;
      }
      const float rs = (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y);
      l = l * alpha + rs;
      m = m_new;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[buf]));
      if (j > 0) {
        if (!accumulate(gj - 1, alpha_prev)) { ok = false; break; }
      }
      alpha_prev = alpha;
    }
    if (ok && n_kv > 0) ok = accumulate(g0 + n_kv - 1, alpha_prev);
    g0 += n_kv > 0 ? n_kv : 0;

    if (ok) {
      // combine the two halves' row sums, normalise and store
      float* xb = xch;  // all earlier exchanges on this buffer were consumed before pair_sync below
      pair_sync(quad);
      xb[half * BLK + r] = l;
      pair_sync(quad);
      const float l_tot = l + xb[(half ^ 1) * BLK + r];
      pair_sync(quad);  // the partner has read this slot before the next item reuses it
      const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
      if (row_g < p.Sq) {
        __nv_bfloat16* op = p.O + (long long)b * p.o_sb + (long long)row_g * p.o_ss +
                            (long long)h * p.o_sh + half * DH;
#pragma unroll
        for (int c8 = 0; c8 < DH / 8; ++c8) {
          uint4 u;
          u.x = pack_bf16x2(o[c8 * 4 + 0].x * inv, o[c8 * 4 + 0].y * inv);
          u.y = pack_bf16x2(o[c8 * 4 + 1].x * inv, o[c8 * 4 + 1].y * inv);
          u.z = pack_bf16x2(o[c8 * 4 + 2].x * inv, o[c8 * 4 + 2].y * inv);
          u.w = pack_bf16x2(o[c8 * 4 + 3].x * inv, o[c8 * 4 + 3].y * inv);
          reinterpret_cast<uint4*>(op)[c8] = u;
        }
        if (half == 0)
          p.lse[((long long)b * p.H + h) * p.Sq + row_g] =
              (l_tot > 0.0f) ? (m + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      }
    }
    }  // work items
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_error(p.err, ERR_MBAR_TIMEOUT, 0xA7F0u);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Pair kernel (no bias / lengths): one CTA owns TWO adjacent 128-row query tiles of one (batch, head), so every K and
// V tile that TMA brings in feeds two products, and the probabilities never touch shared memory:
//   S_t = Q_t·Kᵀ          tcgen05.mma (both operands from shared memory), fp32 in TMEM, one S buffer per query tile
//   P_t = exp2(S_t·c − m)  one softmax warpgroup per query tile, one thread per row; P is written back as bf16 over
//                          the first 64 columns of S_t with tcgen05.st
//   O_t += P_t·V           tcgen05.mma with the A operand read from TMEM; O_t stays in TMEM for the whole item
// The running maximum is only raised when it grew by more than 8 (in the log2 domain): P then stays below 2^8, the
// row sum and O keep one common reference, and the rescale of O_t in TMEM (load, multiply, store) is rare.  The MMA
// warp alternates the two tiles (PV_0, QK_0, PV_1, QK_1, ...), so the tensor pipe works on one tile while the other
// tile's warpgroup is in its softmax.  Shared-memory traffic per query tile and KV tile drops from 224 KB (two
// operand reads per product, K and V written per tile, P written and read) to 128 KB.
// ------------------------------------------------------------------------------------------------------------------
// Phase clocks of CTA 0 (SM cycles summed over the launch), written when tracing is switched on:
//   softmax warp 0:  0 steps, 1 wait for S, 2 S load, 3 maximum / rescale, 4 first half of P, 5 second half of P,
//                    6 output, 7 items
//   MMA thread:      8 PV calls, 9 wait first half of P, 10 wait V, 11 first four PV steps, 12 wait second half,
//                    13 last four PV steps and commits, 14 QK waits (Q, K), 15 QK issue and commits
constexpr int PAIR_TRACE_SLOTS = 16;
__device__ unsigned long long g_pair_trace[PAIR_TRACE_SLOTS];
constexpr int PAIR_THREADS = 384;   // two softmax warpgroups + one warpgroup holding the producer and MMA warps
// Registers are a per-scheduler pool of 512 per lane shared by three warps here (launch allocation 168 each): the
// producer / MMA warpgroup hands its share back and each softmax warp, which keeps a 128-column row of S live, grows.
constexpr int PAIR_REGS_AUX = 88, PAIR_REGS_SOFTMAX = 208;
constexpr int PAIR_STAGES = 4;      // ring of K / V tiles in the order K_j, V_j, K_j+1, V_j+1

template <int D>
struct PairSmem {
  static constexpr int TILE = BLK * D * 2;
  static constexpr int Q_OFF = 0;                          // two query tiles
  static constexpr int KV_OFF = 2 * TILE;
  static constexpr int BAR_OFF = KV_OFF + PAIR_STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 256;
};

template <int D>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using L = PairSmem<D>;
  constexpr int KB = D / 64;
  constexpr uint32_t S_COL = 0;       // S_t at S_COL + 128 t; P_t (bf16 pairs) over its first 64 columns
  constexpr uint32_t O_COL = 256;     // O_t at O_COL + D t
  constexpr uint32_t TMEM_COLS = 512;
  constexpr float RESCALE_STEP = 8.0f;

  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) report_error(p.err, ERR_BOUNDS, 0xA7F3u);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;             // 2
  uint64_t* q_empty = bars + 2;        // 2
  uint64_t* kv_full = bars + 4;        // PAIR_STAGES
  uint64_t* kv_empty = bars + 8;       // PAIR_STAGES
  uint64_t* s_full = bars + 12;        // 2
  uint64_t* p_full = bars + 14;        // 2 (one arrival per softmax warp of the tile)
  uint64_t* o_full = bars + 16;        // 2
  uint64_t* p_half = bars + 18;        // 2: the first 64 columns of P_t are in TMEM (PV starts on them)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hb = p.H * p.B;
  const int n_pairs = (p.n_q + 1) / 2;
  const int n_kv_all = (p.Sk + BLK - 1) / BLK;
  // Items are sorted by decreasing work; round k hands items [k G, (k + 1) G) to the G CTAs in alternating direction
  // (CTA i takes k G + i in even rounds and k G + G - 1 - i in odd ones), which keeps the per-CTA sums within a few
  // percent of each other where a plain stride would leave the first CTAs with the heavy end of every round.
  auto item_of_round = [&](int round) {
    const int G = gridDim.x, i = blockIdx.x;
    return round * G + ((round & 1) ? G - 1 - i : i);
  };
  // Work item w -> (query pair, head, batch) and the KV tiles each of its two query tiles visits
  auto item_at = [&](int w, int& qp, int& h, int& b, int& n0, int& n1) {
    qp = n_pairs - 1 - w / hb;
    const int rem = w % hb;
    h = rem % p.H;
    b = rem / p.H;
    n0 = p.causal ? min(n_kv_all, 2 * qp + 1) : n_kv_all;
    n1 = (2 * qp + 1 < p.n_q) ? (p.causal ? min(n_kv_all, 2 * qp + 2) : n_kv_all) : 0;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&q_full[i]), 1);
      mbar_init(smem_u32(&q_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&p_full[i]), 4);
      mbar_init(smem_u32(&p_half[i]), 4);
      mbar_init(smem_u32(&o_full[i]), 1);
    }
    for (int i = 0; i < PAIR_STAGES; ++i) {
      mbar_init(smem_u32(&kv_full[i]), 1);
      mbar_init(smem_u32(&kv_empty[i]), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PAIR_REGS_AUX));
  if (warp == 8) {
    // ---------------------------- TMA producer ---------------------------------------------------
    if (lane == 0) {
      int g = 0;                 // KV tiles loaded so far over all items: K at ring index 2g, V at 2g + 1
      int items_t[2] = {0, 0};   // items in which query tile t took part (phase of q_full / q_empty)
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = item_of_round(round);
        if (w >= p.n_items) break;
        int qp, h, b, n_t[2];
        item_at(w, qp, h, b, n_t[0], n_t[1]);
        const int n_kv = max(n_t[0], n_t[1]);
        if (n_kv <= 0) continue;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (n_t[t] <= 0) continue;
          // the tile's Q buffer is free once its last QK^T of the previous item has completed
          if (items_t[t] > 0 && !mbar_wait(smem_u32(&q_empty[t]), (items_t[t] - 1) & 1, abort_flag)) { ok = false; break; }
          const uint32_t qb = smem_u32(&q_full[t]);
          mbar_arrive_expect_tx(qb, L::TILE);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_4d(smem_u32(smem + L::Q_OFF + t * L::TILE + kb * (BLK * 128)), &tmQ, qb, kb * 64, h,
                        (2 * qp + t) * BLK, b);
          ++items_t[t];
        }
        for (int j = 0; j < n_kv && ok; ++j, ++g) {
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const int idx = 2 * g + kv;
            const int st = idx % PAIR_STAGES;
            const uint32_t ph = (idx / PAIR_STAGES) & 1;
            if (!mbar_wait(smem_u32(&kv_empty[st]), ph ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t fb = smem_u32(&kv_full[st]);
            mbar_arrive_expect_tx(fb, L::TILE);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem_u32(smem + L::KV_OFF + st * L::TILE + kb * (BLK * 128)), kv == 0 ? &tmK : &tmV, fb,
                          kb * 64, h, j * BLK, b);
          }
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------- MMA issuer -----------------------------------------------------
    // The whole warp walks the schedule in step (every value below is warp-uniform, so the compiler can keep the
    // descriptors in uniform registers, which is where tcgen05.mma reads them) and one elected lane issues.
    {
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BLK, D, false, true);
      int g = 0;
      uint32_t steps_t[2] = {0, 0};   // softmax steps of tile t consumed so far (phase of p_full)
      int items_t[2] = {0, 0};
      int n_t[2] = {0, 0};
      // Descriptor words are formed once: the high word is common to every tile, the low word of a K step is the
      // tile's low word plus a compile-time offset, so an MMA costs a handful of instructions in this single
      // issuing thread (which otherwise, not the tensor pipe, sets the pace).
      constexpr uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t q_lo0 = smem_desc_lo(smem_u32(smem + L::Q_OFF), 16);
      const uint32_t k_lo0 = smem_desc_lo(smem_u32(smem + L::KV_OFF), 16);           // K tiles: K-major
      const uint32_t v_lo0 = smem_desc_lo(smem_u32(smem + L::KV_OFF), BLK * 128);    // V tiles: MN-major
      // The K (V) tile of step j is released by the last product that reads it: tile 1's when tile 1 visits step j.
      const bool tr = p.trace != nullptr && blockIdx.x == 0;
      uint32_t c0 = 0, c1 = 0;
      uint32_t tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      const bool leader = elect_one();
      auto issue_qk = [&](int t, int j) -> bool {
        if (tr) c0 = static_cast<uint32_t>(clock());
        if (j == 0 && !mbar_wait_warp(smem_u32(&q_full[t]), items_t[t] & 1, abort_flag)) return false;
        const int idx = 2 * (g + j);
        const int st = idx % PAIR_STAGES;
        if (!mbar_wait_warp(smem_u32(&kv_full[st]), (idx / PAIR_STAGES) & 1, abort_flag)) return false;
        tc_fence_after();
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[6] += c1 - c0; }
        const uint32_t a_lo = q_lo0 + t * (L::TILE >> 4);
        const uint32_t b_lo = k_lo0 + st * (L::TILE >> 4);
        const uint32_t d_tmem = tmem_u + S_COL + t * BLK;
        if (leader) {
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t off = (kb * (BLK * 128) + k * 32) >> 4;
              umma_bf16_ss_split(d_tmem, a_lo + off, desc_hi, b_lo + off, desc_hi, idesc_s, (kb | k) != 0 ? 1u : 0u);
            }
          umma_commit(smem_u32(&s_full[t]));
          if (t == 1 || j >= n_t[1]) umma_commit(smem_u32(&kv_empty[st]));
          if (j == n_t[t] - 1) umma_commit(smem_u32(&q_empty[t]));
        }
        __syncwarp();
        if (tr) tacc[7] += static_cast<uint32_t>(clock()) - c1;
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        if (tr) c0 = static_cast<uint32_t>(clock());
        if (!mbar_wait_warp(smem_u32(&p_half[t]), steps_t[t] & 1u, abort_flag)) return false;
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[1] += c1 - c0; tacc[0] += 1; c0 = c1; }
        const int idx = 2 * (g + j) + 1;
        const int st = idx % PAIR_STAGES;
        if (!mbar_wait_warp(smem_u32(&kv_full[st]), (idx / PAIR_STAGES) & 1, abort_flag)) return false;
        tc_fence_after();
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[2] += c1 - c0; c0 = c1; }
        const uint32_t b_lo = v_lo0 + st * (L::TILE >> 4);
        const uint32_t a_tmem = tmem_u + S_COL + t * BLK;
        const uint32_t d_tmem = tmem_u + O_COL + t * D;
        // A = P from TMEM (8 columns per K = 16 step); B = V (MN-major: D contiguous, KV rows = K)
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < BLK / 32; ++kk)
            umma_bf16_ts_split(d_tmem, a_tmem + kk * 8, b_lo + ((kk * (16 * 128)) >> 4), desc_hi, idesc_pv,
                               (j | kk) != 0 ? 1u : 0u);
        }
        __syncwarp();
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[3] += c1 - c0; c0 = c1; }
        if (!mbar_wait_warp(smem_u32(&p_full[t]), steps_t[t] & 1u, abort_flag)) return false;   // second half of P_t
        tc_fence_after();
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[4] += c1 - c0; c0 = c1; }
        if (leader) {
#pragma unroll
          for (int kk = BLK / 32; kk < BLK / 16; ++kk)
            umma_bf16_ts_split(d_tmem, a_tmem + kk * 8, b_lo + ((kk * (16 * 128)) >> 4), desc_hi, idesc_pv, 1u);
          if (t == 1 || j >= n_t[1]) umma_commit(smem_u32(&kv_empty[st]));
          if (j == n_t[t] - 1) umma_commit(smem_u32(&o_full[t]));
        }
        __syncwarp();
        ++steps_t[t];
        if (tr) tacc[5] += static_cast<uint32_t>(clock()) - c0;
        return true;
      };
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = item_of_round(round);
        if (w >= p.n_items) break;
        int qp, h, b;
        item_at(w, qp, h, b, n_t[0], n_t[1]);
        const int n_kv = max(n_t[0], n_t[1]);
        if (n_kv <= 0) continue;
        if (n_t[0] > 0) ok = issue_qk(0, 0);
        if (ok && n_t[1] > 0) ok = issue_qk(1, 0);
        for (int j = 0; j < n_kv && ok; ++j) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!ok || j >= n_t[t]) continue;
            ok = issue_pv(t, j);
            if (ok && j + 1 < n_t[t]) ok = issue_qk(t, j + 1);
          }
        }
        g += n_kv;
        if (n_t[0] > 0) ++items_t[0];
        if (n_t[1] > 0) ++items_t[1];
      }
      if (tr && lane == 0)
        for (int i = 0; i < 8; ++i) p.trace[8 + i] += tacc[i];
    }
  }
  } else {
    // ---------------------------- softmax / output warpgroups ------------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PAIR_REGS_SOFTMAX));
    const int t = warp >> 2;              // query tile of the pair
    const int quad = warp & 3;            // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;       // row of the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + S_COL + t * BLK;
    const uint32_t o_addr = tmem_base + lane_off + O_COL + t * D;
    const float sc = p.scale_log2;
    uint32_t steps = 0;   // softmax steps done (phase of s_full)
    int items = 0;        // items this tile took part in (phase of o_full)
    bool ok = true;
    const bool tr = p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    uint32_t c0 = 0, c1 = 0;
    uint32_t tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int round = 0; ok; ++round) {
        const int w = item_of_round(round);
        if (w >= p.n_items) break;
      int qp, h, b, n0, n1;
      item_at(w, qp, h, b, n0, n1);
      const int n_kv = t == 0 ? n0 : n1;
      if (n_kv <= 0) continue;
      const int q_tile = 2 * qp + t;
      const int row_g = q_tile * BLK + r;
      float m = -INFINITY, l = 0.0f;
      for (int j = 0; j < n_kv; ++j) {
        if (tr) c0 = static_cast<uint32_t>(clock());
        if (!mbar_wait_warp(smem_u32(&s_full[t]), steps & 1u, abort_flag)) { ok = false; break; }
        ++steps;
        tc_fence_after();
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[1] += c1 - c0; tacc[0] += 1; c0 = c1; }
        uint32_t sr[BLK];
        {
          uint32_t t0[32], t1[32], t2[32], t3[32];
          tmem_ld_32x32(s_addr, t0);
          tmem_ld_32x32(s_addr + 32, t1);
          tmem_ld_32x32(s_addr + 64, t2);
          tmem_ld_32x32(s_addr + 96, t3);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) { sr[c] = t0[c]; sr[32 + c] = t1[c]; sr[64 + c] = t2[c]; sr[96 + c] = t3[c]; }
        }
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[2] += c1 - c0; c0 = c1; }
        const int col0 = j * BLK;
        float mx = -INFINITY;
        if ((p.causal && j == q_tile) || col0 + BLK > p.Sk) {
#pragma unroll
          for (int c = 0; c < BLK; ++c) {
            const int col = col0 + c;
            const bool dead = (col >= p.Sk) || (p.causal && col > row_g);
            const float s = dead ? -INFINITY : __uint_as_float(sr[c]);
            sr[c] = __float_as_uint(s);
            mx = fmaxf(mx, s);
          }
        } else {
          float mc[8];                                 // eight independent chains
#pragma unroll
          for (int q = 0; q < 8; ++q) mc[q] = fmaxf(__uint_as_float(sr[2 * q]), __uint_as_float(sr[2 * q + 1]));
#pragma unroll
          for (int c = 16; c < BLK; c += 16) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              mc[q] = max3(mc[q], __uint_as_float(sr[c + 2 * q]), __uint_as_float(sr[c + 2 * q + 1]));
          }
          mx = fmaxf(fmaxf(max3(mc[0], mc[1], mc[2]), max3(mc[3], mc[4], mc[5])), fmaxf(mc[6], mc[7]));
        }
        const float m_new = fmaxf(m, mx * sc);
        bool raise = false;
        float alpha = 1.0f;
        if (j == 0) {
          m = m_new;                                   // O_t is overwritten by the first PV: nothing to rescale
        } else if (m_new - m > RESCALE_STEP) {
          raise = true;
          alpha = fast_exp2(m - m_new);                // m = -inf gives 0
          m = m_new;
          l *= alpha;
        }
        if (__any_sync(0xffffffffu, raise)) {
          // S_t of this step was committed after PV_t of the previous step, so O_t is complete here
          const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t v[32];
            tmem_ld_32x32(o_addr + ch * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const float2 y = mul2(make_float2(__uint_as_float(v[2 * c]), __uint_as_float(v[2 * c + 1])), a2);
              v[2 * c] = __float_as_uint(y.x);
              v[2 * c + 1] = __float_as_uint(y.y);
            }
            tmem_st_32x32(o_addr + ch * 32, v);
          }
        }
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[3] += c1 - c0; c0 = c1; }
        const float m_ref = (m == -INFINITY) ? 0.0f : m;
        const float2 sc2 = make_float2(sc, sc);
        const float2 nm2 = make_float2(-m_ref, -m_ref);
        float2 rs2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t pr[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int cc = hlf * 64 + 2 * c;
            const float2 x = fma2(make_float2(__uint_as_float(sr[cc]), __uint_as_float(sr[cc + 1])), sc2, nm2);
            const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            rs2[c & 1] = add2(rs2[c & 1], e);
            pr[c] = pack_bf16x2(e.x, e.y);
          }
          tmem_st_32x32(s_addr + hlf * 32, pr);
          if (hlf == 0) {          // PV_t may start on the first 64 keys while the rest is computed
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_half[t]));
            if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[4] += c1 - c0; c0 = c1; }
          }
        }
        l += (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&p_full[t]));
        if (tr) { c1 = static_cast<uint32_t>(clock()); tacc[5] += c1 - c0; }
      }
      if (!ok) break;
      if (tr) c0 = static_cast<uint32_t>(clock());
      // ---- output: O_t / l as bf16, one row per thread; log-sum-exp in natural units ----
      if (!mbar_wait_warp(smem_u32(&o_full[t]), items & 1, abort_flag)) { ok = false; break; }
      ++items;
      tc_fence_after();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      __nv_bfloat16* op = p.O + (long long)b * p.o_sb + (long long)row_g * p.o_ss + (long long)h * p.o_sh;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t v[32];
        tmem_ld_32x32(o_addr + ch * 32, v);
        tmem_ld_wait();
        if (row_g < p.Sq) {
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[c8 * 8 + 0]) * inv, __uint_as_float(v[c8 * 8 + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(v[c8 * 8 + 2]) * inv, __uint_as_float(v[c8 * 8 + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(v[c8 * 8 + 4]) * inv, __uint_as_float(v[c8 * 8 + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(v[c8 * 8 + 6]) * inv, __uint_as_float(v[c8 * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(op)[ch * 4 + c8] = u;
          }
        }
      }
      if (row_g < p.Sq)
        p.lse[((long long)b * p.H + h) * p.Sq + row_g] =
            (l > 0.0f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      if (tr) { tacc[6] += static_cast<uint32_t>(clock()) - c0; tacc[7] += 1; }
      // the next item's first PV_t overwrites O_t only after this warpgroup's next p_full arrival, which follows
      // these loads in program order
      tc_fence_before();
    }
    if (tr)
      for (int i = 0; i < 8; ++i) p.trace[i] += tacc[i];
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_error(p.err, ERR_MBAR_TIMEOUT, 0xA7F2u);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

namespace st {
// 4-D tensor map over a [B, S, H, D] bf16 view with arbitrary B/S/H strides (D contiguous):
// dims {D, H, S, B}, box {64, 1, rows, 1}.
bool encode_bshd_tmap(CUtensorMap* out, const void* base, int B, int S, int H, int D,
                      long long sb, long long ss, long long sh, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
}
}  // namespace st

struct StAttnFwdArgs {
  const void* Q; const void* K; const void* V; void* O; float* lse;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh;
  int B, H, Sq, Sk, D;
  float scale;
  int causal;
  // optional additive biases (fp32) and valid lengths (int32 [B]); all null = the plain kernel
  const float* key_bias;  long long kb_sb, kb_sh;            // [B, (H,) Sk]
  const float* attn_bias; long long ab_sb, ab_sh, ab_sq;     // [B, (H,) Sq, Sk], keys contiguous
  const int* lengths;
};

// 1 (default): plain attention runs the pair kernel (two query tiles per CTA, P and O in TMEM); 0: the single-tile
// kernel for every case.  The biased / variable-length instantiation always uses the single-tile kernel.
static int g_pair_kernel = 1;
static int g_pair_trace_on = 0;
// Phase tracing of the pair kernel (CTA 0 only; slots listed at g_pair_trace): on = 1 zeroes the sums and makes
// later launches add to them, st_attn_fwd_read_trace copies the 16 sums out after a synchronisation.
ST_API int st_attn_fwd_set_trace(int on) {
  g_pair_trace_on = on ? 1 : 0;
  if (on) {
    unsigned long long zeros[PAIR_TRACE_SLOTS] = {};
    ST_CUDA_CHECK(cudaMemcpyToSymbol(g_pair_trace, zeros, sizeof(zeros)));
  }
  return ST_OK;
}
ST_API int st_attn_fwd_read_trace(unsigned long long* out, int n) {
  if (!out || n < PAIR_TRACE_SLOTS) return st::fail(ST_ERR_INVALID, "attn_fwd_read_trace: need room for 16 values");
  ST_CUDA_CHECK(cudaDeviceSynchronize());
  ST_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_pair_trace, sizeof(unsigned long long) * PAIR_TRACE_SLOTS));
  return ST_OK;
}
ST_API void st_attn_fwd_set_pair_kernel(int on) { g_pair_kernel = on ? 1 : 0; }
ST_API int st_attn_fwd_get_pair_kernel() { return g_pair_kernel; }

ST_API int st_attn_fwd(const StAttnFwdArgs* a, void* stream_v) {
  if (!a || !a->Q || !a->K || !a->V || !a->O || !a->lse) return st::fail(ST_ERR_INVALID, "attn_fwd: null pointer");
  if (a->D != 64 && a->D != 128) return st::fail(ST_ERR_INVALID, "attn_fwd: head_dim must be 64 or 128");
  if (a->causal && a->Sq != a->Sk) return st::fail(ST_ERR_INVALID, "attn_fwd: causal needs seq_q == seq_k");
  const long long strides[] = {a->q_sb, a->q_ss, a->q_sh, a->k_sb, a->k_ss, a->k_sh,
                               a->v_sb, a->v_ss, a->v_sh, a->o_sb, a->o_ss, a->o_sh};
  for (long long s : strides)
    if (s & 7) return st::fail(ST_ERR_INVALID, "attn_fwd: strides must be multiples of 8 elements");
  if ((reinterpret_cast<uintptr_t>(a->Q) | reinterpret_cast<uintptr_t>(a->K) |
       reinterpret_cast<uintptr_t>(a->V) | reinterpret_cast<uintptr_t>(a->O)) & 15)
    return st::fail(ST_ERR_INVALID, "attn_fwd: pointers must be 16-byte aligned");
  CUtensorMap tq, tk, tv;
  if (!st::encode_bshd_tmap(&tq, a->Q, a->B, a->Sq, a->H, a->D, a->q_sb, a->q_ss, a->q_sh, BLK) ||
      !st::encode_bshd_tmap(&tk, a->K, a->B, a->Sk, a->H, a->D, a->k_sb, a->k_ss, a->k_sh, BLK) ||
      !st::encode_bshd_tmap(&tv, a->V, a->B, a->Sk, a->H, a->D, a->v_sb, a->v_ss, a->v_sh, BLK))
    return ST_ERR_CUDA;
  AttnFwdParams p;
  p.O = static_cast<__nv_bfloat16*>(a->O);
  p.lse = a->lse;
  p.o_sb = a->o_sb; p.o_ss = a->o_ss; p.o_sh = a->o_sh;
  p.B = a->B; p.H = a->H; p.Sq = a->Sq; p.Sk = a->Sk;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.causal = a->causal;
  p.err = st::error_word();
  p.n_q = (a->Sq + BLK - 1) / BLK;
  p.n_items = p.n_q * a->H * a->B;
  p.key_bias = a->key_bias; p.kb_sb = a->kb_sb; p.kb_sh = a->kb_sh;
  p.attn_bias = a->attn_bias; p.ab_sb = a->ab_sb; p.ab_sh = a->ab_sh; p.ab_sq = a->ab_sq;
  p.lengths = a->lengths;
  p.trace = nullptr;
  const bool biased = a->key_bias || a->attn_bias || a->lengths;
  if (p.n_items <= 0) return ST_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (!biased && g_pair_kernel) {
    // two query tiles per CTA: the items are (query pair, head, batch)
    if (g_pair_trace_on) ST_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.trace), g_pair_trace));
    p.n_items = ((p.n_q + 1) / 2) * a->H * a->B;
    const dim3 pgrid(std::min(p.n_items, st::sm_count()));
    const int dev = st::current_device();
    auto plaunch = [&](auto kern, int smem_bytes, bool* cfg) -> int {
      if (!cfg[dev]) {
        ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        cfg[dev] = true;
      }
      kern<<<pgrid, PAIR_THREADS, smem_bytes, s>>>(tq, tk, tv, p);
      return ST_OK;
    };
    static bool pcfg[2][st::kMaxDevices] = {{false}};
    const int prc = a->D == 128 ? plaunch(attn_fwd_pair_kernel<128>, PairSmem<128>::TOTAL, pcfg[0])
                                : plaunch(attn_fwd_pair_kernel<64>, PairSmem<64>::TOTAL, pcfg[1]);
    if (prc != ST_OK) return prc;
    ST_CUDA_CHECK(cudaGetLastError());
    return ST_OK;
  }
  // persistent: one CTA per SM walks the work items, so TMEM, barriers and the pipeline fill are
  // paid once per CTA and an item's output stores overlap the next item's first loads
  const dim3 grid(std::min(p.n_items, st::sm_count()));
  auto launch = [&](auto kern, int smem_bytes, bool* cfg) -> int {
    if (!cfg[st::current_device()]) {     // the attribute is per device
      ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
      cfg[st::current_device()] = true;
    }
    kern<<<grid, NUM_THREADS, smem_bytes, s>>>(tq, tk, tv, p);
    return ST_OK;
  };
  static bool cfg[4][st::kMaxDevices] = {{false}};
  int rc;
  if (a->D == 128) {
    rc = biased ? launch(attn_fwd_kernel<128, true>, FwdSmem<128>::TOTAL, cfg[0])
                : launch(attn_fwd_kernel<128, false>, FwdSmem<128>::TOTAL, cfg[1]);
  } else {
    rc = biased ? launch(attn_fwd_kernel<64, true>, FwdSmem<64>::TOTAL, cfg[2])
                : launch(attn_fwd_kernel<64, false>, FwdSmem<64>::TOTAL, cfg[3]);
  }
  if (rc != ST_OK) return rc;
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
