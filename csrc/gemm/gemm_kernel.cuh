// The persistent tcgen05 GEMM kernel, shared by the plain launcher (gemm_sm100.cu) and the
// tensor-parallel launchers (csrc/comm/tp_gemm.cu).
//
// COMM selects what else the launch does:
//   COMM_NONE  C = epilogue(alpha * A·Bᵀ)
//   COMM_AG    all-gather → GEMM.  A is the gathered activation [T, K].  Every CTA of the launch
//              has two extra warps that push a 1/gridDim slice of this rank's shard into every
//              rank's gather buffer (bulk copies through a small shared-memory ring, plain peer
//              writes over NVLink, destinations in ring order) and count per-sub-chunk arrivals,
//              while its other warps run GEMM tiles.  The TMA producer waits (bounded) for the
//              counter of the rows it is about to load; the local rows are read from the shard
//              itself; tiles are ordered local chunk first, then in ring order.
//   COMM_RS    GEMM → reduce-scatter.  Tiles are ordered so that the chunk this rank owns comes last (or, with
//              row-block groups, so that each group of the own chunk comes one group after the remote tiles of
//              the same group: see map_tile).
//              For the other chunks the epilogue TMA-stores each partial tile straight into the
//              owner's staging slot (peer writes over NVLink) and counts the tile on the owner's
//              per-row-block counter.  For its own chunk the epilogue waits (bounded) until every
//              peer's partial of the row block has landed, adds them and the optional residual to
//              the accumulator in fp32, and writes the final bf16 rows — there is no separate
//              reduction pass and the local partial is never staged.
#pragma once
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../comm/comm.cuh"

namespace st {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int NUM_THREADS_AG = 256;  // all-gather variant: + warp 6 (shard push) and warp 7 (arrival publisher)
constexpr int AG_RING_CHUNK = 16384;  // bytes per bulk copy of the push ring
constexpr int AG_RING_SLOTS = 3;      // the ring sits behind the barriers of the 3-stage GEMM layout

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_GELU_BWD = 3, ACT_RELU_BWD = 4 };
enum Comm : int { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2 };
constexpr int kMaxSubChunks = 16;   // arrival counters reserved per source rank (AG)

struct GemmComm {
  PeerGroup g;
  int rows_per_chunk;   // rows owned by each rank (T / world), multiple of BM
  int sub_per_chunk;    // arrival-flag granularity (AG): sub-chunks per rank shard
  int gemm_ctas;        // CTAs that run GEMM tiles; CTAs beyond them only push (AG)
  int slot_enter;       // entry rendezvous slot (world words)
  // ---- AG ----
  const __nv_bfloat16* src_shard;          // [rows_per_chunk, K] contiguous
  __nv_bfloat16* gather_peers[kMaxRanks];  // [T, K] contiguous on every rank
  __nv_bfloat16* gather_mc;                // multicast alias or null
  int slot_arrive;      // arrival words: slot_arrive + src * kMaxSubChunks + sub
  unsigned arrive_target;  // value an arrival word must reach: the epoch (peer-store path, one
                           // writer per word) or a cumulative count (multicast path, n_comm writers)
  unsigned long long* trace;  // optional [gridDim.x][4] globaltimer stamps (start, entry, tiles/push done, end)
  int sub_major;        // tile order of the remote chunks: 0 chunk by chunk (ring), 1 sub-chunk by sub-chunk
  int local_in_place;   // AG: the shard already lives in this rank's slot of its own gather buffer (no local copy)
  int rs_groups;        // RS: row-block groups per chunk; remote and local tiles are interleaved group by group
  int rs_lag;           // RS: groups a local group trails the remote group of the same index (>= 1)
  // ---- RS ----
  __nv_bfloat16* stage_peers[kMaxRanks];   // on each owner: [world][rows_per_chunk, N]
  int slot_done;        // counters: slot_done + row block within the chunk
  unsigned done_target; // counter value meaning "every rank's tiles of this row block landed"
  __nv_bfloat16* rs_out;                   // [rows_per_chunk, N] reduced local shard
  const __nv_bfloat16* rs_residual;        // optional, added during the reduction
};

// Implicit-GEMM convolution (3x3, stride 1, padding 1, NHWC activations).
//   mode 1 (forward / data gradient): the A tile of 128 output pixels is a 4-D TMA box
//          {64 channels, W, Hb, Nb} taken at the tap's (kh-1, kw-1) offset; pixels outside the image
//          are zero-filled by TMA.  K = 9 * C runs tap-major, matching weights stored [OC][tap][C].
//   mode 2 (weight gradient): K runs over pixels; the B tile (64 pixels x 64-channel blocks of the
//          shifted input) is the 4-D box, A is dYᵀ; the batch index enumerates (tap, K split).
struct ConvGeom {
  int mode;
  int H, W;          // image size
  int Hb, Nb;        // rows / images per pixel block (mode 1: 128 pixels, mode 2: 64 pixels)
  int c_chunks;      // input channels / 64 (mode 1)
  int taps;          // 9
};

struct GemmParams {
  ConvGeom conv;
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
  int batch;
  long long batch_stride_c;
  int use_tma_store;   // bf16 output without accumulation: stage through smem, store by TMA
  unsigned* err;
};

// Tensor maps of the output: [0] for a plain GEMM, one per owner rank for GEMM → reduce-scatter.
struct OutMaps {
  CUtensorMap m[kMaxRanks];
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int CSTAGE_OFFSET = STAGES * STAGE_BYTES;       // 4 warps x 2 buffers x 4 KiB
  static constexpr int CSTAGE_BYTES = 4 * 2 * 4096;
  static constexpr int BAR_OFFSET = CSTAGE_OFFSET + CSTAGE_BYTES;
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

// Tile index → (batch, tm, tn); with a communication plan the M dimension is walked chunk by
// chunk in ring order (`chunk_shift` = 0 starts at the local chunk, 1 ends with it).
template <int COMM>
__device__ __forceinline__ void map_tile(int t, int tiles_m, int tiles_n, int tiles_per_batch,
                                         const GemmComm& c, int& b, int& tm, int& tn) {
  if constexpr (COMM == COMM_NONE) {
    b = t / tiles_per_batch;
    tile_coords(t - b * tiles_per_batch, tiles_m, tiles_n, tm, tn);
  } else {
    b = 0;
    const int tiles_m_chunk = c.rows_per_chunk / BM;
    const int per_chunk = tiles_m_chunk * tiles_n;
    if (COMM == COMM_AG && c.sub_major && t >= per_chunk) {
      // remote rows: for every sub-chunk index, the W-1 remote chunks in ring order
      const int msub = tiles_m_chunk / c.sub_per_chunk;       // M tiles per sub-chunk
      const int per_sub = msub * tiles_n;
      const int r = t - per_chunk;
      const int blk = r / per_sub;
      const int s = blk / (c.g.world - 1);
      const int ci = 1 + blk % (c.g.world - 1);
      const int rr = r - blk * per_sub;
      tn = rr / msub;
      tm = ((c.g.rank + ci) % c.g.world) * tiles_m_chunk + s * msub + rr % msub;
      return;
    }
    if (COMM == COMM_RS && c.rs_groups > 1) {
      // Row blocks of every chunk are split into G groups.  Order (lag 1): R(0), R(1), L(0), R(2), L(1), ...,
      // R(G-1), L(G-2), L(G-1), where R(g) are the tiles of group g of the W-1 remote chunks (ring order) and
      // L(g) the tiles of group g of this rank's own chunk.  A local tile needs every peer's partial of its row
      // block; peers deliver those in their R(g), so running L(g) `lag` groups late lets the final reduction of
      // group g ride behind later transfers instead of after all of them.  lag >= G is "all remote, then local".
      const int W = c.g.world, G = c.rs_groups;
      const int lag = min(max(c.rs_lag, 1), G);          // local group g runs after remote group g + lag
      const int msub = tiles_m_chunk / G;
      const int per_l = msub * tiles_n;
      const int per_r = (W - 1) * per_l;
      int g, r;
      bool local;
      if (t < lag * per_r) {                             // R(0) .. R(lag-1)
        g = per_r > 0 ? t / per_r : 0; local = false; r = t - g * per_r;
      } else {
        const int u = t - lag * per_r;
        const int pairs = G - lag;                       // (R(lag + i), L(i)) for i < pairs
        if (u < pairs * (per_r + per_l)) {
          const int pair = u / (per_r + per_l);
          const int v = u - pair * (per_r + per_l);
          if (v < per_r) { g = lag + pair; local = false; r = v; }
          else { g = pair; local = true; r = v - per_r; }
        } else {                                         // L(pairs) .. L(G-1)
          const int w = u - pairs * (per_r + per_l);
          g = pairs + w / per_l; local = true; r = w - (w / per_l) * per_l;
        }
      }
      int lm;
      if (local) {
        tile_coords(r, msub, tiles_n, lm, tn);
        tm = c.g.rank * tiles_m_chunk + g * msub + lm;
      } else {
        const int ci = r / per_l;
        tile_coords(r - ci * per_l, msub, tiles_n, lm, tn);
        tm = ((c.g.rank + 1 + ci) % W) * tiles_m_chunk + g * msub + lm;
      }
      return;
    }
    const int ci = t / per_chunk;
    int lm;
    tile_coords(t - ci * per_chunk, tiles_m_chunk, tiles_n, lm, tn);
    const int shift = (COMM == COMM_AG) ? 0 : 1;
    const int chunk = (c.g.rank + shift + ci) % c.g.world;
    tm = chunk * tiles_m_chunk + lm;
  }
}

// ---- reduce-scatter: sources added to a tile of the rows this rank owns ----------------------
constexpr int kRsBatch = 4;   // sources whose loads are in flight together (4 x 64 B per lane each)

__device__ __forceinline__ void prefetch_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

// Source s of the local reduction: the staged partials of the other ranks in rank order (this
// rank's own slot is skipped), then the residual.
__device__ __forceinline__ const __nv_bfloat16* rs_src(const GemmComm& cm, int s, long long slot_stride) {
  const int q = s + (s >= cm.g.rank ? 1 : 0);
  return q < cm.g.world ? cm.stage_peers[cm.g.rank] + q * slot_stride
                        : cm.rs_residual;
}

__device__ __forceinline__ void rs_load_batch(const GemmComm& cm, long long slot_stride, int s0, int n_srcs, long long off,
                                              uint4 (&buf)[kRsBatch][4]) {
#pragma unroll
  for (int i = 0; i < kRsBatch; ++i) {
    if (s0 + i < n_srcs) {
      const uint4* sp = reinterpret_cast<const uint4*>(rs_src(cm, s0 + i, slot_stride) + off);
#pragma unroll
      for (int k = 0; k < 4; ++k) buf[i][k] = sp[k];
    }
  }
}

__device__ __forceinline__ void rs_add_batch(int s0, int n_srcs, const uint4 (&buf)[kRsBatch][4], float* v) {
#pragma unroll
  for (int i = 0; i < kRsBatch; ++i) {
    if (s0 + i < n_srcs) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f0 = unpack_bf16x2(buf[i][k].x), f1 = unpack_bf16x2(buf[i][k].y), f2 = unpack_bf16x2(buf[i][k].z),
               f3 = unpack_bf16x2(buf[i][k].w);
        v[k * 8 + 0] += f0.x; v[k * 8 + 1] += f0.y; v[k * 8 + 2] += f1.x; v[k * 8 + 3] += f1.y;
        v[k * 8 + 4] += f2.x; v[k * 8 + 5] += f2.y; v[k * 8 + 6] += f3.x; v[k * 8 + 7] += f3.y;
      }
    }
  }
}

__device__ __forceinline__ void epilogue_bar() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int COMM>
__global__ void __launch_bounds__(COMM == COMM_AG ? NUM_THREADS_AG : NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ OutMaps tmC, const __grid_constant__ CUtensorMap tmA_local,
                 const GemmParams p, const GemmComm cm) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int gemm_bid = blockIdx.x;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = tiles_m * tiles_n;
  const int total_tiles = tiles_per_batch * p.batch;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int grid_stride = gridDim.x;
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
    if constexpr (COMM == COMM_AG) {
      tmem_slot[2] = 0;   // items whose stores are complete (push warp → publisher warp)
      tmem_slot[3] = 0;   // push warp has finished
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if constexpr (COMM == COMM_RS) {
      // tell every peer that this rank has left the previous launch that used the staging area
      if (blockIdx.x == 0) {
        fence_sys();
        for (int q = 0; q < cm.g.world; ++q)
          st_relaxed_sys(cm.g.signals[q] + cm.slot_enter + cm.g.rank, cm.g.epoch);
      }
    }
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
      for (int t = gemm_bid; t < total_tiles && ok; t += grid_stride) {
        int b, tm, tn;
        map_tile<COMM>(t, tiles_m, tiles_n, tiles_per_batch, cm, b, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const CUtensorMap* mapA = &tmA;
        int m_coord = m0;
        if constexpr (COMM == COMM_AG) {
          const int src = m0 / cm.rows_per_chunk;
          const int sub = (m0 - src * cm.rows_per_chunk) / (cm.rows_per_chunk / cm.sub_per_chunk);
          if (src == cm.g.rank) {
            // the local rows are read from the shard itself; nothing to wait for
            mapA = &tmA_local;
            m_coord = m0 - src * cm.rows_per_chunk;
          } else if (!wait_flag_ge(cm.g.signals[cm.g.rank] + cm.slot_arrive + src * kMaxSubChunks + sub,
                                   cm.arrive_target)) {
            *abort_flag = 1;
            report_error(p.err, ERR_FLAG_TIMEOUT, 0xA601u);
            break;
          }
          fence_proxy_async_global();
        }
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
          if (p.conv.mode == 1) {
            // A: 128 output pixels (Nb images x Hb rows x W) shifted by the tap, 64 channels
            const int tap = kb / p.conv.c_chunks, cc = kb - tap * p.conv.c_chunks;
            const int hblocks = p.conv.H / p.conv.Hb;
            const int img0 = (tm / hblocks) * p.conv.Nb, h0 = (tm % hblocks) * p.conv.Hb;
            tma_load_4d(sa, mapA, fb, cc * 64, tap % 3 - 1, h0 + tap / 3 - 1, img0);
            tma_load_3d(sb, &tmB, fb, k0, n0, 0);
          } else if (p.conv.mode == 2) {
            // batch index = tap + taps * split; K block = 64 consecutive pixels
            const int tap = b % p.conv.taps, split = b / p.conv.taps;
            const int kg = split * k_blocks + kb;                  // global pixel block
            const int hblocks = p.conv.H / p.conv.Hb;
            const int img0 = (kg / hblocks) * p.conv.Nb, h0 = (kg % hblocks) * p.conv.Hb;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * (64 * BK * 2), mapA, fb, m_coord + 64 * j, kg * BK, 0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_4d(sb + j * (64 * BK * 2), &tmB, fb, n0 + 64 * j, tap % 3 - 1, h0 + tap / 3 - 1, img0);
          } else {
            if constexpr (!A_MN) {
              tma_load_3d(sa, mapA, fb, k0, m_coord, b);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_3d(sa + j * (64 * BK * 2), mapA, fb, m_coord + 64 * j, k0, b);
            }
            if constexpr (!B_MN) {
              tma_load_3d(sb, &tmB, fb, k0, n0, b);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * (64 * BK * 2), &tmB, fb, n0 + 64 * j, k0, b);
            }
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
      for (int t = gemm_bid; t < total_tiles && ok; t += grid_stride, ++iter) {
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
  } else if (warp < 6) {
    // ------------------------------- epilogue warps -----------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int iter = 0;
    // staging buffers per warp: two, except in the 4-stage all-gather variant, whose push ring takes
    // the upper half of the staging area
    constexpr int CSB = (COMM == COMM_AG && STAGES == 4) ? 1 : 2;
    int store_seq = 0;          // TMA stores issued by this warp (selects the staging buffer)
    int tile_seq0 = 0;          // value of store_seq when the current tile started
    constexpr int kPubBatch = 3;
    int pend_owner[kPubBatch], pend_block[kPubBatch], n_pend = 0;   // RS: tiles stored, not yet published
    bool alive = true;
    bool saw_local = false;     // RS tracing: the first local tile has been stamped
    const bool tracer = (COMM != COMM_NONE) && cm.trace && quad == 2 && lane == 0;   // warp 2
    if (tracer) cm.trace[blockIdx.x * 4 + 0] = globaltimer_ns();
    if constexpr (COMM == COMM_RS) {
      // peers' staging areas are free once every peer has entered this launch
      bool ok = true;
      if (lane == 0)
        for (int q = 0; q < cm.g.world && ok; ++q)
          ok = wait_flag_ge(cm.g.signals[cm.g.rank] + cm.slot_enter + q, cm.g.epoch);
      alive = __all_sync(0xffffffffu, ok);
      if (!alive) {
        *abort_flag = 1;
        if (lane == 0) report_error(p.err, ERR_FLAG_TIMEOUT, 0xA602u);
      }
    }
    if (tracer) cm.trace[blockIdx.x * 4 + 1] = globaltimer_ns();
    for (int t = gemm_bid; t < total_tiles && alive; t += grid_stride, ++iter) {
      int b, tm, tn;
      map_tile<COMM>(t, tiles_m, tiles_n, tiles_per_batch, cm, b, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait_warp(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag)) break;
      tc_fence_after();
      tile_seq0 = store_seq;
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      void* c_ptr = p.C;
      const int cbatch = (p.conv.mode == 2) ? (b % p.conv.taps) : b;
      long long c_base = (long long)cbatch * p.batch_stride_c + (long long)row * p.ldc;
      int owner = 0;
      bool local_tile = false;
      int n_srcs = 0;             // RS local tile: staged partials + residual to add
      long long red_off = 0;      // element offset of this lane's row segment inside a source
      bool pf_valid = false;      // pf holds the first batch of the next column group
      uint4 pf[kRsBatch][4];
      const long long slot_stride = (long long)cm.rows_per_chunk * p.ldc;
      if constexpr (COMM == COMM_RS) {
        owner = m0 / cm.rows_per_chunk;
        local_tile = owner == cm.g.rank;
        if (local_tile) {
          if (tracer && !saw_local) cm.trace[(gridDim.x + blockIdx.x) * 4 + 0] = globaltimer_ns();
          // Everything this warp still owes its peers is published first: they wait for it before
          // they can finish, exactly as this rank is about to wait for them.
          if (lane == 0 && n_pend > 0) {
            if (p.use_tma_store) tma_store_wait<0>();
            fence_proxy_async_global();
            fence_sys();
            for (int i = 0; i < n_pend; ++i)
              red_relaxed_sys_add(cm.g.signals[pend_owner[i]] + cm.slot_done + pend_block[i], 1u);
            n_pend = 0;
          }
          // this rank owns these rows: wait until every peer's partial of the row block has landed,
          // then the column loop adds them (and the residual) and writes the final rows
          bool okc = true;
          if (lane == 0)
            okc = wait_flag_ge(cm.g.signals[cm.g.rank] + cm.slot_done + (m0 - owner * cm.rows_per_chunk) / BM,
                               cm.done_target);
          okc = __all_sync(0xffffffffu, okc);
          if (!okc) {
            *abort_flag = 1;
            if (lane == 0) report_error(p.err, ERR_FLAG_TIMEOUT, 0xA603u);
            break;
          }
          c_ptr = cm.rs_out;
          c_base = (long long)(row - owner * cm.rows_per_chunk) * p.ldc;
          if (tracer && !saw_local) {
            saw_local = true;
            cm.trace[(gridDim.x + blockIdx.x) * 4 + 1] = globaltimer_ns();
          }
          // Sources to add: the other ranks' staged partials (slot q of this rank's staging area), then
          // the residual.  The whole row segment goes to L2 now; the first batch of the first column
          // group is loaded before the accumulator is read, and every later group's first batch is
          // loaded while the previous group is converted and stored.
          n_srcs = cm.g.world - 1 + (cm.rs_residual ? 1 : 0);
          red_off = c_base + n0;
          if (row_ok) {
            const int lines = (min(BN, p.N - n0) * 2 + 127) / 128;
            for (int s_ = 0; s_ < n_srcs; ++s_)
              for (int l_ = 0; l_ < lines; ++l_) prefetch_l2(rs_src(cm, s_, slot_stride) + red_off + l_ * 64);
            pf_valid = n0 + 32 <= p.N;
            if (pf_valid) rs_load_batch(cm, slot_stride, 0, n_srcs, red_off, pf);
          }
        } else {
          c_ptr = cm.stage_peers[owner];
          c_base = ((long long)cm.g.rank * cm.rows_per_chunk + (row - owner * cm.rows_per_chunk)) * p.ldc;
        }
      }
      // TMA mode: after the second half of a 64-column chunk (or the last valid half) one lane
      // hands the warp's staged 32 x 64 block to the copy engine
      auto issue_store = [&](int c, int col0) {
        if ((c & 1) == 0 && col0 + 32 < p.N) return;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const CUtensorMap* om = &tmC.m[COMM == COMM_RS ? owner : 0];
          const int r0 = (COMM == COMM_RS ? m0 - owner * cm.rows_per_chunk : m0) + quad * 32;
          tma_store_3d(om, smem_u32(smem + L::CSTAGE_OFFSET + (quad * CSB + (store_seq % CSB)) * 4096),
                       n0 + (c >> 1) * 64, r0, b);
          tma_store_commit();
        }
        ++store_seq;
      };
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        if (p.use_tma_store && (c & 1) == 0 && store_seq >= CSB) {
          // the staging buffer about to be rewritten was handed to TMA CSB stores ago
          if (lane == 0) tma_store_wait_read<CSB - 1>();
          __syncwarp();
        }
        if (!row_ok) {
          // rows past M: nothing to compute; in TMA mode the warp still issues its store
          // (the copy clips rows and columns that fall outside the tensor)
          if (p.use_tma_store) issue_store(c, col0);
          continue;
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const bool full = (col0 + 32 <= p.N);
        if constexpr (COMM == COMM_RS) {
          if (local_tile) {
            const long long off = red_off + c * 32;
            if (full) {
              if (!pf_valid) rs_load_batch(cm, slot_stride, 0, n_srcs, off, pf);
              rs_add_batch(0, n_srcs, pf, v);
              for (int s0 = kRsBatch; s0 < n_srcs; s0 += kRsBatch) {
                uint4 more[kRsBatch][4];
                rs_load_batch(cm, slot_stride, s0, n_srcs, off, more);
                rs_add_batch(s0, n_srcs, more, v);
              }
              pf_valid = (c + 1 < BN / 32) && (col0 + 64 <= p.N);
              if (pf_valid) rs_load_batch(cm, slot_stride, 0, n_srcs, off + 32, pf);
            } else {
              pf_valid = false;
              for (int s_ = 0; s_ < n_srcs; ++s_) {
                const __nv_bfloat16* src = rs_src(cm, s_, slot_stride) + off;
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) v[j] += __bfloat162float(src[j]);
              }
            }
          }
        }
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
        if (p.use_tma_store) {
          // stage this warp's 32 rows x 64 columns (128-byte swizzle) and store them by TMA
          const int half = c & 1;
          uint8_t* cs = smem + L::CSTAGE_OFFSET + (quad * CSB + (store_seq % CSB)) * 4096;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
            *reinterpret_cast<uint4*>(cs + sw128_offset(lane, half * 4 + q)) = o;
          }
        } else if (p.out_fp32) {
          float* cp = reinterpret_cast<float*>(c_ptr) + c_base + col0;
          if (full && (p.ldc & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (p.accumulate == 2) {  // split-K: several CTAs add into the same tile
                atomicAdd(reinterpret_cast<float4*>(cp) + q, o);
                continue;
              }
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
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(c_ptr) + c_base + col0;
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
        if (p.use_tma_store) issue_store(c, col0);
      }
      // hand the accumulator back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      if constexpr (COMM == COMM_RS) {
        // Publish this warp's 32 rows to the owner (the counter counts warp arrivals, so no
        // CTA-wide barrier is needed).  Waiting for the stores of the tile just issued would put
        // an NVLink round trip into every tile, and so would a system-scope release per tile:
        // finished tiles are queued and published kPubBatch at a time behind one fence, after
        // the wait that leaves only the newest tile's store groups outstanding.
        if (lane == 0 && !local_tile) {
          if (p.use_tma_store) {
            if (n_pend == kPubBatch) {
              const int groups = store_seq - tile_seq0;      // bulk groups committed for this tile
              switch (groups) {
                case 0: tma_store_wait<0>(); break;
                case 1: tma_store_wait<1>(); break;
                case 2: tma_store_wait<2>(); break;
                case 3: tma_store_wait<3>(); break;
                default: tma_store_wait<4>(); break;
              }
              fence_proxy_async_global();
              fence_sys();
              for (int i = 0; i < n_pend; ++i)
                red_relaxed_sys_add(cm.g.signals[pend_owner[i]] + cm.slot_done + pend_block[i], 1u);
              n_pend = 0;
            }
            pend_owner[n_pend] = owner;
            pend_block[n_pend] = (m0 - owner * cm.rows_per_chunk) / BM;
            ++n_pend;
          } else {
            red_release_sys_add(cm.g.signals[owner] + cm.slot_done + (m0 - owner * cm.rows_per_chunk) / BM, 1u);
          }
        }
      }
    }
    if (p.use_tma_store && lane == 0) tma_store_wait<0>();
    if (tracer) cm.trace[blockIdx.x * 4 + 2] = globaltimer_ns();
    if constexpr (COMM == COMM_RS) {
      if (lane == 0 && n_pend > 0) {
        fence_proxy_async_global();
        fence_sys();
        for (int i = 0; i < n_pend; ++i)
          red_relaxed_sys_add(cm.g.signals[pend_owner[i]] + cm.slot_done + pend_block[i], 1u);
      }
    }

  } else if constexpr (COMM == COMM_AG) {
    // ---------------------------------------------------------------------------------------
    // All-gather: EVERY CTA pushes its 1/gridDim slice of this rank's shard while its other warps
    // run GEMM tiles (one SM sustains only ~20 GB/s of peer writes, so the push is spread over
    // all of them instead of a few dedicated CTAs).  A work item is one sub-chunk for one
    // destination; items go destination-major in ring order (rank-1, rank-2, ..., own buffer
    // last), so in every phase the W senders address W different receivers and a receiver gets
    // the chunks in the order its GEMM tiles consume them.  Warp 6 lane 0 drives bulk copies
    // local HBM → shared-memory ring → destination; warp 7 lane 0 adds one arrival per finished
    // item to the destination's counter, so the system-scope release never stalls the copies.
    // ---------------------------------------------------------------------------------------
    volatile int* s_done_items = reinterpret_cast<volatile int*>(tmem_slot + 2);
    volatile int* s_finished = reinterpret_cast<volatile int*>(tmem_slot + 3);
    const int W = cm.g.world, R = cm.g.rank;
    const int SUBS = cm.sub_per_chunk;
    // the copy into this rank's own gather buffer comes last and is skipped when the shard already lives there
    const int items = (cm.local_in_place ? W - 1 : W) * SUBS;
    auto dest_of = [&](int item) {
      const int q = item / SUBS;
      return q < W - 1 ? (R - 1 - q + W) % W : R;
    };
    if (warp == 7 && lane == 0) {
      int sent = 0;
      const uint64_t t0 = globaltimer_ns();
      for (;;) {
        const int fin = *s_finished;
        const int d = *s_done_items;
        if (sent < d) {
          // one fence for everything that completed since the last look, then plain atomics
          __threadfence_block();
          fence_proxy_async_global();
          fence_sys();
          for (; sent < d; ++sent)
            red_relaxed_sys_add(cm.g.signals[dest_of(sent)] + cm.slot_arrive + R * kMaxSubChunks + sent % SUBS, 1u);
        }
        if (sent >= items || (fin && sent >= *s_done_items)) break;
        if (globaltimer_ns() - t0 > (uint64_t)(W + 2) * wait_limit_ns()) break;   // the copy thread reports the cause
        __nanosleep(64);
      }
    } else if (warp == 6 && lane == 0) {
      bool ok = true;
      if (cm.trace) cm.trace[(gridDim.x + blockIdx.x) * 4 + 0] = globaltimer_ns();
      if (blockIdx.x == 0) {
        fence_sys();
        for (int q = 0; q < W; ++q) st_relaxed_sys(cm.g.signals[q] + cm.slot_enter + R, cm.g.epoch);
      }
      // peers must have left the previous launch that read this gather buffer
      for (int q = 0; q < W && ok; ++q) ok = wait_flag_ge(cm.g.signals[R] + cm.slot_enter + q, cm.g.epoch);
      if (cm.trace) cm.trace[(gridDim.x + blockIdx.x) * 4 + 1] = globaltimer_ns();
      if (!ok) {
        report_error(p.err, ERR_FLAG_TIMEOUT, 0xA600u);
      } else {
        // 3-stage variant (communication-bound shapes): 3 x 16 KB behind the barriers; 4-stage variant
        // (compute-bound shapes): 2 x 8 KB in the upper half of the output staging area
        constexpr int NB = (STAGES == 4) ? 2 : AG_RING_SLOTS;
        constexpr uint32_t CH = (STAGES == 4) ? 8192 : AG_RING_CHUNK;
        uint8_t* ring = (STAGES == 4) ? smem + L::CSTAGE_OFFSET + 16384 : smem + L::BAR_OFFSET + 256;
        uint64_t* cbar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET + 128);
        const long long sub_bytes = (long long)(cm.rows_per_chunk / SUBS) * p.K * 2;
        long long slice = (sub_bytes + gridDim.x - 1) / gridDim.x;
        slice = (slice + 127) & ~127ll;
        const long long lo = min(sub_bytes, (long long)blockIdx.x * slice);
        const long long hi = min(sub_bytes, lo + slice);
        const int n_ch = (int)((hi - lo + CH - 1) / CH);     // chunks per item for this CTA (may be 0)
        if (n_ch == 0 || items == 0) {
          *s_done_items = items;                              // nothing to copy: the arrivals still count
        } else {
          volatile int local_abort = 0;
          for (int i = 0; i < NB; ++i) mbar_init(smem_u32(&cbar[i]), 1);
          fence_barrier_init();
          const char* src_base = reinterpret_cast<const char*>(cm.src_shard);
          const long long dst_base = (long long)R * cm.rows_per_chunk * p.K * 2;
          const int total = items * n_ch;
          auto chunk_of = [&](int c, int& item, uint32_t& sz) {
            item = c / n_ch;
            const long long o = lo + (long long)(c - item * n_ch) * CH;
            sz = (uint32_t)min((long long)CH, hi - o);
            return (long long)(item % SUBS) * sub_bytes + o;
          };
          auto issue_load = [&](int c) {
            int item;
            uint32_t sz;
            const long long off = chunk_of(c, item, sz);
            const int b = c % NB;
            mbar_arrive_expect_tx(smem_u32(&cbar[b]), sz);
            bulk_load_g2s(smem_u32(ring + b * CH), src_base + off, sz, smem_u32(&cbar[b]));
          };
          // one load ahead of the store being issued; a buffer is reloaded once the store that
          // used it has finished reading shared memory (NB - 1 stores may be in flight)
          issue_load(0);
          uint32_t phase_bits = 0;
          for (int c = 0; c < total; ++c) {
            const int b = c % NB;
            if (c + 1 < total) {
              if (c + 1 >= NB) tma_store_wait_read<NB - 2>();   // store c + 1 - NB has released its buffer
              issue_load(c + 1);
            }
            if (!mbar_wait(smem_u32(&cbar[b]), (phase_bits >> b) & 1u, &local_abort)) { ok = false; break; }
            phase_bits ^= (1u << b);
            int item;
            uint32_t sz;
            const long long off = chunk_of(c, item, sz);
            bulk_store_s2g(reinterpret_cast<char*>(cm.gather_peers[dest_of(item)]) + dst_base + off,
                           smem_u32(ring + b * CH), sz);
            tma_store_commit();
            if (c >= NB - 1) {
              tma_store_wait<NB - 1>();                       // every store up to chunk c - (NB - 1) is complete
              const int cc = c - (NB - 1);
              if (cc % n_ch == n_ch - 1) {
                fence_proxy_async_global();
                __threadfence_block();
                *s_done_items = cc / n_ch + 1;
                if (cm.trace && cc / n_ch + 1 == (W - 1) * SUBS)     // every remote store of this CTA has completed
                  cm.trace[(2 * gridDim.x + blockIdx.x) * 4 + 0] = globaltimer_ns();
              }
            }
          }
          tma_store_wait<0>();
          if (!ok) {
            report_error(p.err, ERR_MBAR_TIMEOUT, 0xA604u);
          } else {
            fence_proxy_async_global();
            __threadfence_block();
            *s_done_items = items;
          }
        }
      }
      if (cm.trace) cm.trace[(gridDim.x + blockIdx.x) * 4 + 2] = globaltimer_ns();
      __threadfence_block();
      *s_finished = 1;
    }
  }

  // ------------------------------- teardown -------------------------------------------
  if constexpr (COMM != COMM_NONE) {
    if (cm.trace && threadIdx.x == 64) cm.trace[blockIdx.x * 4 + 3] = globaltimer_ns();
  }
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

}  // namespace gemm
}  // namespace st
