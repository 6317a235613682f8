// Whole-sequence recurrent scans: ONE launch runs every time step of an Elman (tanh), wave-gated (dilated
// skip) or LSTM layer, forward or backward-through-time, instead of a Python loop of per-step launches.
//
//   forward   z_t = zx_t + hin_t · W_hh,  hin_t = h_{t-1} (+ h_{t-d} for the wave cell),  h_t = cell(z_t)
//   backward  dz_t = cell'(·) ∘ dh_t,  dhin_t = dz_t · W_hhᵀ flows to h_{t-1} (and h_{t-d})
//
// The input projection zx = x · W_ih + b for all steps, and the parameter gradients
// dW_hh = hinᵀ · dz, dW_ih = xᵀ · dz, dx = dz · W_ihᵀ, are single tcgen05 GEMMs over [B·T] rows issued by the
// caller; only the part that is sequential in t lives here.  Batch rows are independent, so a CTA owns RB
// rows for the whole sequence: W_hh sits in shared memory (fp32, row stride padded by one word so that both
// the forward column walk and the backward row walk are conflict-free), thread j owns gate column j.
//
// Reference parity: lstm_forward_gate_step / lstm_backward_scan.wgsl, wave_gate_project / wave_gate_backward
// (crates/st-tensor/src/wgpu_shaders), layers crates/st-nn/src/layers/{spiral_rnn,wave_rnn,lstm}.rs.
#include "../common/host.h"

namespace {

constexpr int RB = 4;                    // batch rows per CTA
enum Cell : int { CELL_TANH = 0, CELL_WAVE = 1, CELL_LSTM = 2 };

struct ScanParams {
  const float* zx;      // [B, T, G*H]   input projection + bias
  const float* w_hh;    // [H, G*H]
  float* h_all;         // [B, T, H]     h_t
  float* hin_all;       // [B, T, H]     recurrent input of step t (h_{t-1} + skip)
  float* z_all;         // [B, T, G*H]   tanh / wave: pre-activations; lstm: activated gates (i|f|g|o)
  float* c_all;         // [B, T, H]     lstm cell state (null otherwise)
  // backward only
  const float* dh_last; // [B, H]        gradient of the last hidden state
  float* dz_all;        // [B, T, G*H]
  float* dhin_all;      // [B, T, H]     scratch: gradient of hin_t
  int B, T, H, G, cell, dilation;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

__global__ void __launch_bounds__(1024)
rnn_scan_fwd_kernel(const ScanParams p) {
  extern __shared__ float sm[];
  const int H = p.H, GH = p.G * p.H, ldw = GH + 1;
  float* Wsm = sm;                       // [H][GH + 1]
  float* hin = Wsm + (size_t)H * ldw;    // [RB][H]
  float* zbuf = hin + RB * H;            // [RB][GH]
  const int j = threadIdx.x;             // gate column
  const int b0 = blockIdx.x * RB;
  for (int i = threadIdx.x; i < H * GH; i += blockDim.x) Wsm[(i / GH) * ldw + i % GH] = p.w_hh[i];
  for (int i = threadIdx.x; i < RB * H; i += blockDim.x) hin[i] = 0.0f;
  float c_state[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) c_state[r] = 0.0f;
  __syncthreads();
  for (int t = 0; t < p.T; ++t) {
    if (j < GH) {
      float acc[RB];
#pragma unroll
      for (int r = 0; r < RB; ++r)
        acc[r] = (b0 + r < p.B) ? p.zx[((size_t)(b0 + r) * p.T + t) * GH + j] : 0.0f;
      for (int k = 0; k < H; ++k) {
        const float w = Wsm[k * ldw + j];
#pragma unroll
        for (int r = 0; r < RB; ++r) acc[r] = fmaf(hin[r * H + k], w, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < RB; ++r) zbuf[r * GH + j] = acc[r];
    }
    __syncthreads();
    if (j < H) {
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const int b = b0 + r;
        if (b >= p.B) continue;
        const size_t row = (size_t)b * p.T + t;
        p.hin_all[row * H + j] = hin[r * H + j];
        float h;
        if (p.cell == CELL_TANH) {
          const float z = zbuf[r * GH + j];
          p.z_all[row * GH + j] = z;
          h = tanhf(z);
        } else if (p.cell == CELL_WAVE) {
          const float za = zbuf[r * GH + j], zb = zbuf[r * GH + H + j];
          p.z_all[row * GH + j] = za;
          p.z_all[row * GH + H + j] = zb;
          h = tanhf(za) * sigmoidf_(zb);
        } else {
          const float gi = sigmoidf_(zbuf[r * GH + j]), gf = sigmoidf_(zbuf[r * GH + H + j]);
          const float gg = tanhf(zbuf[r * GH + 2 * H + j]), go = sigmoidf_(zbuf[r * GH + 3 * H + j]);
          c_state[r] = gf * c_state[r] + gi * gg;
          h = go * tanhf(c_state[r]);
          float* a = p.z_all + row * GH;
          a[j] = gi; a[H + j] = gf; a[2 * H + j] = gg; a[3 * H + j] = go;
          p.c_all[row * H + j] = c_state[r];
        }
        p.h_all[row * H + j] = h;
        // recurrent input of the next step: h_t, plus for the wave cell the output of step (t + 1) - dilation,
        // which this same thread wrote earlier (or is writing now when dilation == 1)
        float nxt = h;
        if (p.cell == CELL_WAVE && t + 1 >= p.dilation) {
          const int ts = t + 1 - p.dilation;
          nxt += (ts == t) ? h : p.h_all[((size_t)b * p.T + ts) * H + j];
        }
        hin[r * H + j] = nxt;
      }
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024)
rnn_scan_bwd_kernel(const ScanParams p) {
  extern __shared__ float sm[];
  const int H = p.H, GH = p.G * p.H, ldw = GH + 1;
  float* Wsm = sm;                       // [H][GH + 1]
  float* dzbuf = Wsm + (size_t)H * ldw;  // [RB][GH]
  const int j = threadIdx.x;
  const int b0 = blockIdx.x * RB;
  for (int i = threadIdx.x; i < H * GH; i += blockDim.x) Wsm[(i / GH) * ldw + i % GH] = p.w_hh[i];
  float dc[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) dc[r] = 0.0f;
  __syncthreads();
  for (int t = p.T - 1; t >= 0; --t) {
    if (j < H) {
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const int b = b0 + r;
        if (b >= p.B) {
          for (int g = 0; g < p.G; ++g) dzbuf[r * GH + g * H + j] = 0.0f;
          continue;
        }
        const size_t row = (size_t)b * p.T + t;
        // dh_t: the loss gradient of the last state, what step t+1 sent back through its recurrent input and,
        // for the wave cell, what step t+dilation sent back through its skip input (written by this thread)
        float dh = (t == p.T - 1) ? p.dh_last[(size_t)b * H + j] : p.dhin_all[(row + 1) * H + j];
        if (p.cell == CELL_WAVE && t + p.dilation < p.T && !(p.dilation == 1 && t == p.T - 1))
          dh += p.dhin_all[(row + p.dilation) * H + j];
        if (p.cell == CELL_TANH) {
          const float h = p.h_all[row * H + j];
          const float dz = dh * (1.0f - h * h);
          dzbuf[r * GH + j] = dz;
          p.dz_all[row * GH + j] = dz;
        } else if (p.cell == CELL_WAVE) {
          const float ta = tanhf(p.z_all[row * GH + j]), sb = sigmoidf_(p.z_all[row * GH + H + j]);
          const float da = dh * sb * (1.0f - ta * ta), db = dh * ta * sb * (1.0f - sb);
          dzbuf[r * GH + j] = da; dzbuf[r * GH + H + j] = db;
          p.dz_all[row * GH + j] = da; p.dz_all[row * GH + H + j] = db;
        } else {
          const float* a = p.z_all + row * GH;
          const float gi = a[j], gf = a[H + j], gg = a[2 * H + j], go = a[3 * H + j];
          const float c = p.c_all[row * H + j];
          const float c_prev = t > 0 ? p.c_all[(row - 1) * H + j] : 0.0f;
          const float tc = tanhf(c);
          const float dct = dh * go * (1.0f - tc * tc) + dc[r];
          const float d0 = dct * gg * gi * (1.0f - gi), d1 = dct * c_prev * gf * (1.0f - gf);
          const float d2 = dct * gi * (1.0f - gg * gg), d3 = dh * tc * go * (1.0f - go);
          dc[r] = dct * gf;
          dzbuf[r * GH + j] = d0; dzbuf[r * GH + H + j] = d1; dzbuf[r * GH + 2 * H + j] = d2; dzbuf[r * GH + 3 * H + j] = d3;
          float* o = p.dz_all + row * GH;
          o[j] = d0; o[H + j] = d1; o[2 * H + j] = d2; o[3 * H + j] = d3;
        }
      }
    }
    __syncthreads();
    if (j < H) {
      // dhin_t[r][j] = sum_g dz_t[r][g] * W_hh[j][g]  (row j of W_hh)
      float acc[RB];
#pragma unroll
      for (int r = 0; r < RB; ++r) acc[r] = 0.0f;
      for (int g = 0; g < GH; ++g) {
        const float w = Wsm[j * ldw + g];
#pragma unroll
        for (int r = 0; r < RB; ++r) acc[r] = fmaf(dzbuf[r * GH + g], w, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < RB; ++r)
        if (b0 + r < p.B) p.dhin_all[((size_t)(b0 + r) * p.T + t) * H + j] = acc[r];
    }
    __syncthreads();
  }
}

int smem_bytes(int H, int G) { return (int)(((size_t)H * (G * H + 1) + (size_t)RB * H + (size_t)RB * G * H) * sizeof(float)); }

}  // namespace

struct StRnnScanArgs {
  const float* zx; const float* w_hh;
  float* h_all; float* hin_all; float* z_all; float* c_all;
  const float* dh_last; float* dz_all; float* dhin_all;
  int B, T, H, cell, dilation, backward;
};

// 1 when the whole-sequence kernel takes this layer (gate columns fit one CTA, W_hh fits shared memory).
ST_API int st_rnn_scan_supported(int H, int cell) {
  const int G = cell == CELL_TANH ? 1 : (cell == CELL_WAVE ? 2 : 4);
  return (H > 0 && G * H <= 1024 && smem_bytes(H, G) <= 200 * 1024) ? 1 : 0;
}

ST_API int st_rnn_scan(const StRnnScanArgs* a, void* stream_v) {
  if (!a || !a->zx || !a->w_hh || !a->h_all || !a->hin_all || !a->z_all)
    return st::fail(ST_ERR_INVALID, "rnn_scan: null pointer");
  if (a->cell < CELL_TANH || a->cell > CELL_LSTM) return st::fail(ST_ERR_INVALID, "rnn_scan: unknown cell");
  if (a->cell == CELL_LSTM && !a->c_all) return st::fail(ST_ERR_INVALID, "rnn_scan: lstm needs c_all");
  if (a->B <= 0 || a->T <= 0) return st::fail(ST_ERR_INVALID, "rnn_scan: empty input");
  if (a->cell == CELL_WAVE && a->dilation < 1) return st::fail(ST_ERR_INVALID, "rnn_scan: dilation must be >= 1");
  if (!st_rnn_scan_supported(a->H, a->cell)) return st::fail(ST_ERR_TOO_LARGE, "rnn_scan: hidden size too large for the one-CTA scan");
  if (a->backward && (!a->dh_last || !a->dz_all || !a->dhin_all)) return st::fail(ST_ERR_INVALID, "rnn_scan: backward needs dh_last, dz_all, dhin_all");
  ScanParams p;
  p.zx = a->zx; p.w_hh = a->w_hh; p.h_all = a->h_all; p.hin_all = a->hin_all; p.z_all = a->z_all; p.c_all = a->c_all;
  p.dh_last = a->dh_last; p.dz_all = a->dz_all; p.dhin_all = a->dhin_all;
  p.B = a->B; p.T = a->T; p.H = a->H; p.cell = a->cell; p.dilation = a->dilation;
  p.G = a->cell == CELL_TANH ? 1 : (a->cell == CELL_WAVE ? 2 : 4);
  const int GH = p.G * p.H;
  const int threads = ((GH + 31) / 32) * 32;
  const int smem = smem_bytes(p.H, p.G);
  const int grid = (a->B + RB - 1) / RB;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  static int cfg_f[st::kMaxDevices] = {0}, cfg_b[st::kMaxDevices] = {0};   // opted-in bytes, per device
  const int dev = st::current_device();
  if (a->backward) {
    if (smem > cfg_b[dev]) {
      ST_CUDA_CHECK(cudaFuncSetAttribute(rnn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      cfg_b[dev] = smem;
    }
    rnn_scan_bwd_kernel<<<grid, threads, smem, s>>>(p);
  } else {
    if (smem > cfg_f[dev]) {
      ST_CUDA_CHECK(cudaFuncSetAttribute(rnn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      cfg_f[dev] = smem;
    }
    rnn_scan_fwd_kernel<<<grid, threads, smem, s>>>(p);
  }
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
