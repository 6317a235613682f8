// Data-parallel bucket step in ONE kernel: reduce-scatter of the gradient bucket over
// NVLink (NVLS multimem.ld_reduce when a multicast mapping exists, plain peer loads
// otherwise) → gradient scale (1/world, loss scale, clip coefficient) → AdamW or
// SGD-momentum on the shard this rank owns (fp32 master weights and moments are sharded,
// ZeRO-1 style) → all-gather of the updated bf16 weights (multimem.st or peer stores) →
// gradient bucket zeroed for the next step.
//
// Synchronisation: an entry rendezvous (every rank's gradients are final — guaranteed
// locally by stream order, signalled to peers by CTA 0), and an exit rendezvous after the
// last CTA of each rank has pushed its weights (peers may read my gradients until then, and
// nobody may use the new weights earlier).  All waits are bounded; on expiry the kernel
// writes the error word and returns without touching the remaining data.
// The grid never exceeds the SM count, so every CTA is resident while it waits.
//
// Global-norm clipping needs the norm of the whole reduced gradient before any weight moves, so the step can also
// run in two phases per bucket: phase 1 (overlapped with the backward pass) reduces the owned shard, keeps the
// reduced gradient in a shard-sized fp32 buffer and adds its squared norm to a device word; phase 2 (after the
// backward pass) exchanges the ranks' partial norms through a small symmetric array behind its entry rendezvous,
// derives the clip coefficient min(1, max_norm / ||g||) in the kernel and then updates and broadcasts as above.
//
// Reference parity: replaces the per-parameter all-reduce-mean followed by apply_step of
// ModuleTrainer::step (crates/st-nn/src/trainer.rs:7259-7268, :9035-9062) and the thread
// rendezvous all-reduce (crates/spiral-selfsup/src/trainer/distributed.rs:299-430).
#include "../common/host.h"
#include "comm.cuh"

namespace {
using namespace st;

struct DpStepArgs {
  PeerGroup g;
  float* grad_local;                 // this rank's gradient bucket (symmetric), n floats
  const float* grad_mc;              // multicast alias or null
  const float* grad_peers[kMaxRanks];
  __nv_bfloat16* w_local;            // this rank's bf16 weights bucket (symmetric)
  __nv_bfloat16* w_mc;               // multicast alias or null
  __nv_bfloat16* w_peers[kMaxRanks];
  float* master;                     // shard-local fp32 master weights (n / world)
  float* m;                          // Adam first moment / SGD momentum (shard-local)
  float* v;                          // Adam second moment (shard-local, null for SGD)
  long long n;                       // bucket elements, multiple of 8 * world
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, momentum;
  float grad_scale;                  // includes 1/world
  const float* scale_ptr;            // optional device scalar multiplied in (clip coefficient)
  int kind;                          // 0 AdamW, 1 SGD-momentum
  int slot_enter, slot_exit;         // signal slots (each `world` words wide)
  unsigned* cta_counter;             // local counter for "last CTA done"
  unsigned* err;
  // ---- two-phase mode (global-norm clipping) ----
  int phase;                         // 0 one pass; 1 reduce + squared norm; 2 clip + update + broadcast
  float* gred;                       // shard-local reduced gradient (n / world floats), phases 1 and 2
  float* sumsq_local;                // this rank's sum of squares over its shards of every bucket
  float* norm_peers[kMaxRanks];      // symmetric [world] floats: slot r = rank r's sum of squares
  float max_norm;                    // clip threshold (phase 2)
};

__global__ void __launch_bounds__(512)
dp_step_kernel(const DpStepArgs a) {
  __shared__ int s_ok;
  __shared__ float s_clip;
  __shared__ float s_red[16];
  const int W = a.g.world, R = a.g.rank;
  // ---- entry rendezvous -------------------------------------------------------------------
  if (threadIdx.x == 0) {
    bool ok = true;
    if (a.phase == 2 && blockIdx.x == 0) {
      // this rank's partial norm is final (stream order): hand it to every rank before the entry signal
      const float mine = *a.sumsq_local;
      for (int p = 0; p < W; ++p) a.norm_peers[p][R] = mine;
    }
    if (W > 1) {
      if (blockIdx.x == 0) {
        fence_sys();
        for (int p = 0; p < W; ++p) st_relaxed_sys(a.g.signals[p] + a.slot_enter + R, a.g.epoch);
      }
      for (int p = 0; p < W && ok; ++p) ok = wait_flag_ge(a.g.signals[R] + a.slot_enter + p, a.g.epoch);
    }
    s_ok = ok ? 1 : 0;
    if (a.phase == 2 && ok) {
      // W == 1: the slot was written by CTA 0 of this launch, which other CTAs cannot wait for - read the word itself
      float total = 0.0f;
      if (W == 1) total = *a.sumsq_local;
      else for (int p = 0; p < W; ++p) total += reinterpret_cast<volatile float*>(a.norm_peers[R])[p];
      const float norm = sqrtf(fmaxf(total, 0.0f));
      s_clip = (a.max_norm > 0.0f && norm > a.max_norm) ? a.max_norm / (norm + 1e-6f) : 1.0f;
    }
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) report_error(a.err, ERR_FLAG_TIMEOUT, 0xD900u);
    return;
  }

  // ---- owned shard: reduce, update, broadcast ------------------------------------------------
  const long long shard = a.n / W;
  const long long base = shard * R;
  // phase 2 reads gradients that phase 1 already scaled: only the clip coefficient is left to apply
  const float gs = a.phase == 2 ? s_clip : a.grad_scale * (a.scale_ptr ? *a.scale_ptr : 1.0f);
  float sq = 0.0f;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8; i < shard;
       i += (long long)gridDim.x * blockDim.x * 8) {
    float g[8];
    if (a.phase == 2) {
      const float4 x0 = reinterpret_cast<const float4*>(a.gred + i)[0], x1 = reinterpret_cast<const float4*>(a.gred + i)[1];
      g[0] = x0.x; g[1] = x0.y; g[2] = x0.z; g[3] = x0.w; g[4] = x1.x; g[5] = x1.y; g[6] = x1.z; g[7] = x1.w;
    } else if (a.grad_mc) {
      float4 x0 = multimem_ld_reduce_f32x4(a.grad_mc + base + i);
      float4 x1 = multimem_ld_reduce_f32x4(a.grad_mc + base + i + 4);
      g[0] = x0.x; g[1] = x0.y; g[2] = x0.z; g[3] = x0.w; g[4] = x1.x; g[5] = x1.y; g[6] = x1.z; g[7] = x1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.0f;
      for (int p = 0; p < W; ++p) {
        const int q = (R + p) % W;  // start with the local copy, stagger the peers
        const float4* src = reinterpret_cast<const float4*>(a.grad_peers[q] + base + i);
        float4 x0 = src[0], x1 = src[1];
        g[0] += x0.x; g[1] += x0.y; g[2] += x0.z; g[3] += x0.w; g[4] += x1.x; g[5] += x1.y; g[6] += x1.z; g[7] += x1.w;
      }
    }
    if (a.phase == 1) {
      // keep the reduced (scaled, not yet clipped) gradient and its squared norm; weights move in phase 2
#pragma unroll
      for (int j = 0; j < 8; ++j) { g[j] *= gs; sq = fmaf(g[j], g[j], sq); }
      reinterpret_cast<float4*>(a.gred + i)[0] = make_float4(g[0], g[1], g[2], g[3]);
      reinterpret_cast<float4*>(a.gred + i)[1] = make_float4(g[4], g[5], g[6], g[7]);
      continue;
    }
    float w[8];
    {
      float4 m0 = reinterpret_cast<float4*>(a.master + i)[0], m1 = reinterpret_cast<float4*>(a.master + i)[1];
      w[0] = m0.x; w[1] = m0.y; w[2] = m0.z; w[3] = m0.w; w[4] = m1.x; w[5] = m1.y; w[6] = m1.z; w[7] = m1.w;
    }
    float mo[8], vo[8];
    {
      float4 a0 = reinterpret_cast<float4*>(a.m + i)[0], a1 = reinterpret_cast<float4*>(a.m + i)[1];
      mo[0] = a0.x; mo[1] = a0.y; mo[2] = a0.z; mo[3] = a0.w; mo[4] = a1.x; mo[5] = a1.y; mo[6] = a1.z; mo[7] = a1.w;
    }
    if (a.kind == 0) {
      float4 b0 = reinterpret_cast<float4*>(a.v + i)[0], b1 = reinterpret_cast<float4*>(a.v + i)[1];
      vo[0] = b0.x; vo[1] = b0.y; vo[2] = b0.z; vo[3] = b0.w; vo[4] = b1.x; vo[5] = b1.y; vo[6] = b1.z; vo[7] = b1.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = g[j] * gs;
        mo[j] = a.beta1 * mo[j] + (1.0f - a.beta1) * gj;
        vo[j] = a.beta2 * vo[j] + (1.0f - a.beta2) * gj * gj;
        w[j] -= a.lr * ((mo[j] / a.bc1) / (sqrtf(vo[j] / a.bc2) + a.eps) + a.weight_decay * w[j]);
      }
      reinterpret_cast<float4*>(a.v + i)[0] = make_float4(vo[0], vo[1], vo[2], vo[3]);
      reinterpret_cast<float4*>(a.v + i)[1] = make_float4(vo[4], vo[5], vo[6], vo[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = g[j] * gs + a.weight_decay * w[j];
        mo[j] = a.momentum * mo[j] + gj;
        w[j] -= a.lr * mo[j];
      }
    }
    reinterpret_cast<float4*>(a.m + i)[0] = make_float4(mo[0], mo[1], mo[2], mo[3]);
    reinterpret_cast<float4*>(a.m + i)[1] = make_float4(mo[4], mo[5], mo[6], mo[7]);
    reinterpret_cast<float4*>(a.master + i)[0] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(a.master + i)[1] = make_float4(w[4], w[5], w[6], w[7]);
    uint4 wb;
    wb.x = pack_bf16x2(w[0], w[1]); wb.y = pack_bf16x2(w[2], w[3]);
    wb.z = pack_bf16x2(w[4], w[5]); wb.w = pack_bf16x2(w[6], w[7]);
    if (a.w_mc) {
      multimem_st_v4(a.w_mc + base + i, wb);
    } else {
      for (int p = 0; p < W; ++p) {
        const int q = (R + p) % W;
        *reinterpret_cast<uint4*>(a.w_peers[q] + base + i) = wb;
      }
    }
  }

  if (a.phase == 1) {
    // block sum of the squared norm, one atomic per CTA
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.0f;
      v = warp_sum(v);
      if (threadIdx.x == 0) atomicAdd(a.sumsq_local, v);
    }
  }

  // ---- exit rendezvous ---------------------------------------------------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok = true;
    if (W > 1) {
      fence_sys();
      const unsigned done = atomicAdd(a.cta_counter, 1u);
      if (done == gridDim.x - 1) {
        *a.cta_counter = 0;  // every CTA of this launch has already counted itself
        fence_sys();
        for (int p = 0; p < W; ++p) st_relaxed_sys(a.g.signals[p] + a.slot_exit + R, a.g.epoch);
      }
      for (int p = 0; p < W && ok; ++p) ok = wait_flag_ge(a.g.signals[R] + a.slot_exit + p, a.g.epoch);
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) report_error(a.err, ERR_FLAG_TIMEOUT, 0xD901u);
    return;
  }
  if (a.phase == 2) return;          // the gradients were consumed and cleared in phase 1
  // every peer has finished reading my gradients: clear the whole local bucket
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < a.n;
       i += (long long)gridDim.x * blockDim.x * 4)
    *reinterpret_cast<float4*>(a.grad_local + i) = z;
}

}  // namespace

struct StPeerGroup {
  int world, rank;
  unsigned epoch;
  unsigned long long signals[st::kMaxRanks];
  unsigned long long signals_mc;
};

struct StDpStepArgs {
  StPeerGroup g;
  unsigned long long grad_local, grad_mc, grad_peers[st::kMaxRanks];
  unsigned long long w_local, w_mc, w_peers[st::kMaxRanks];
  unsigned long long master, m, v;
  long long n;
  float lr, beta1, beta2, eps, weight_decay, momentum;
  int step;
  float grad_scale;
  unsigned long long scale_ptr;
  int kind;
  int slot_enter, slot_exit;
  unsigned long long cta_counter;
  int max_ctas;
  // two-phase mode for global-norm clipping (phase 0 = the single fused pass, all fields below unused)
  int phase;                              // 1: reduce + squared norm into gred / sumsq_local; 2: clip + update + broadcast
  unsigned long long gred;                // fp32 [n / world] reduced gradient of this bucket's owned shard
  unsigned long long sumsq_local;         // fp32 word, zeroed by the caller at the start of the step
  unsigned long long norm_peers[st::kMaxRanks];   // symmetric fp32 [world] on every rank
  float max_norm;
};

namespace st {
void fill_peer_group(PeerGroup& g, const StPeerGroup& s) {
  g.world = s.world;
  g.rank = s.rank;
  g.epoch = s.epoch;
  for (int i = 0; i < kMaxRanks; ++i) g.signals[i] = reinterpret_cast<unsigned*>(s.signals[i]);
  g.signals_mc = reinterpret_cast<unsigned*>(s.signals_mc);
}
}  // namespace st

ST_API int st_dp_step(const StDpStepArgs* s, void* stream_v) {
  if (!s) return st::fail(ST_ERR_INVALID, "dp_step: null args");
  if (s->g.world < 1 || s->g.world > st::kMaxRanks || s->g.rank < 0 || s->g.rank >= s->g.world)
    return st::fail(ST_ERR_INVALID, "dp_step: bad world/rank");
  if (s->n <= 0 || s->n % (8ll * s->g.world) != 0)
    return st::fail(ST_ERR_INVALID, "dp_step: bucket length must be a positive multiple of 8*world");
  if ((s->grad_local | s->w_local | s->master | s->m) == 0 || (s->kind == 0 && s->v == 0))
    return st::fail(ST_ERR_INVALID, "dp_step: null buffer");
  DpStepArgs a;
  st::fill_peer_group(a.g, s->g);
  a.grad_local = reinterpret_cast<float*>(s->grad_local);
  a.grad_mc = reinterpret_cast<const float*>(s->grad_mc);
  a.w_local = reinterpret_cast<__nv_bfloat16*>(s->w_local);
  a.w_mc = reinterpret_cast<__nv_bfloat16*>(s->w_mc);
  for (int i = 0; i < st::kMaxRanks; ++i) {
    a.grad_peers[i] = reinterpret_cast<const float*>(s->grad_peers[i]);
    a.w_peers[i] = reinterpret_cast<__nv_bfloat16*>(s->w_peers[i]);
  }
  a.master = reinterpret_cast<float*>(s->master);
  a.m = reinterpret_cast<float*>(s->m);
  a.v = reinterpret_cast<float*>(s->v);
  a.n = s->n;
  a.lr = s->lr; a.beta1 = s->beta1; a.beta2 = s->beta2; a.eps = s->eps;
  a.weight_decay = s->weight_decay; a.momentum = s->momentum;
  a.bc1 = 1.0f - powf(s->beta1, (float)s->step);
  a.bc2 = 1.0f - powf(s->beta2, (float)s->step);
  a.grad_scale = s->grad_scale;
  a.scale_ptr = reinterpret_cast<const float*>(s->scale_ptr);
  a.kind = s->kind;
  a.slot_enter = s->slot_enter; a.slot_exit = s->slot_exit;
  a.cta_counter = reinterpret_cast<unsigned*>(s->cta_counter);
  a.err = st::error_word();
  a.phase = s->phase;
  a.gred = reinterpret_cast<float*>(s->gred);
  a.sumsq_local = reinterpret_cast<float*>(s->sumsq_local);
  for (int i = 0; i < st::kMaxRanks; ++i) a.norm_peers[i] = reinterpret_cast<float*>(s->norm_peers[i]);
  a.max_norm = s->max_norm;
  if (s->phase < 0 || s->phase > 2) return st::fail(ST_ERR_INVALID, "dp_step: phase must be 0, 1 or 2");
  if (s->phase != 0 && (!s->gred || !s->sumsq_local || !s->norm_peers[s->g.rank]))
    return st::fail(ST_ERR_INVALID, "dp_step: the two-phase mode needs gred, sumsq_local and norm_peers");
  const int threads = 512;
  long long want = (s->n / s->g.world / 8 + threads - 1) / threads;
  int cap = st::sm_count();
  if (s->max_ctas > 0 && s->max_ctas < cap) cap = s->max_ctas;
  int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  dp_step_kernel<<<grid, threads, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(a);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
