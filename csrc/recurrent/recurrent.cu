// Recurrent-cell element-wise kernels (fp32): the LSTM gate step with its backward (one BPTT step),
// the wave gate (tanh·sigmoid) with its backward, and the gather / scatter of the last time step.
//
// Arithmetic restated from the reference's tensor-utility compute shaders
// (crates/st-tensor/src/wgpu_shaders/tensor_utils.wgsl: lstm_forward_gate_step,
// wave_gate_project / wave_gate_backward, sequence_last_step_gather / scatter) and
// lstm_backward_scan.wgsl; the matrix products around them run on the GEMM kernel.
//
//   forward :  z = [i | f | g | o]  (pre-activations, [B, 4H])
//              c' = σ(f)·c + σ(i)·tanh(g),   h' = σ(o)·tanh(c')
//   backward:  given dh', dc' (gradient flowing into c' from the next step) →
//              dz [B, 4H] and dc (gradient flowing to the previous cell state)
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

__global__ void lstm_gate_fwd_kernel(const float* __restrict__ z, const float* __restrict__ c_prev,
                                     float* __restrict__ c_out, float* __restrict__ h_out,
                                     float* __restrict__ act /* [B,4H] activated gates, may be null */, int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / H), j = (int)(idx - (long long)b * H);
    const float* zr = z + (long long)b * 4 * H;
    const float i = sigmoidf_(zr[j]), f = sigmoidf_(zr[H + j]), g = tanhf(zr[2 * H + j]), o = sigmoidf_(zr[3 * H + j]);
    const float c = f * c_prev[idx] + i * g;
    c_out[idx] = c;
    h_out[idx] = o * tanhf(c);
    if (act) {
      float* ar = act + (long long)b * 4 * H;
      ar[j] = i; ar[H + j] = f; ar[2 * H + j] = g; ar[3 * H + j] = o;
    }
  }
}

__global__ void lstm_gate_bwd_kernel(const float* __restrict__ act, const float* __restrict__ c_prev,
                                     const float* __restrict__ c, const float* __restrict__ dh,
                                     const float* __restrict__ dc_next /* may be null */, float* __restrict__ dz,
                                     float* __restrict__ dc_prev, int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / H), j = (int)(idx - (long long)b * H);
    const float* ar = act + (long long)b * 4 * H;
    const float i = ar[j], f = ar[H + j], g = ar[2 * H + j], o = ar[3 * H + j];
    const float tc = tanhf(c[idx]);
    const float dct = dh[idx] * o * (1.0f - tc * tc) + (dc_next ? dc_next[idx] : 0.0f);
    float* dr = dz + (long long)b * 4 * H;
    dr[j] = dct * g * i * (1.0f - i);
    dr[H + j] = dct * c_prev[idx] * f * (1.0f - f);
    dr[2 * H + j] = dct * i * (1.0f - g * g);
    dr[3 * H + j] = dh[idx] * tc * o * (1.0f - o);
    dc_prev[idx] = dct * f;
  }
}

// z = [a | b] ([B, 2H]):  y = tanh(a)·σ(b)
__global__ void wave_gate_fwd_kernel(const float* __restrict__ z, float* __restrict__ y, int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / H), j = (int)(idx - (long long)b * H);
    const float* zr = z + (long long)b * 2 * H;
    y[idx] = tanhf(zr[j]) * sigmoidf_(zr[H + j]);
  }
}

__global__ void wave_gate_bwd_kernel(const float* __restrict__ z, const float* __restrict__ dy, float* __restrict__ dz,
                                     int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / H), j = (int)(idx - (long long)b * H);
    const float* zr = z + (long long)b * 2 * H;
    const float t = tanhf(zr[j]), s = sigmoidf_(zr[H + j]);
    float* dr = dz + (long long)b * 2 * H;
    dr[j] = dy[idx] * s * (1.0f - t * t);
    dr[H + j] = dy[idx] * t * s * (1.0f - s);
  }
}

// x: [B, steps*dim] → y[B, dim] = last step (gather), or the transposed scatter into a zeroed dx
__global__ void last_step_kernel(const float* __restrict__ src, float* __restrict__ dst, int B, int steps, int dim,
                                 int scatter) {
  const long long n = (long long)B * dim;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / dim), j = (int)(idx - (long long)b * dim);
    const long long wide = ((long long)b * steps + (steps - 1)) * dim + j;
    if (scatter) dst[wide] = src[idx];
    else dst[idx] = src[wide];
  }
}

int grid_for(long long n) {
  long long g = (n + 255) / 256;
  const long long cap = (long long)st::sm_count() * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

ST_API int st_lstm_gate_fwd(const float* z, const float* c_prev, float* c_out, float* h_out, float* act, int B, int H,
                            void* stream) {
  if (!z || !c_prev || !c_out || !h_out || B <= 0 || H <= 0) return st::fail(ST_ERR_INVALID, "lstm_gate_fwd: bad arguments");
  lstm_gate_fwd_kernel<<<grid_for((long long)B * H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(z, c_prev, c_out, h_out,
                                                                                                       act, B, H);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_lstm_gate_bwd(const float* act, const float* c_prev, const float* c, const float* dh, const float* dc_next,
                            float* dz, float* dc_prev, int B, int H, void* stream) {
  if (!act || !c_prev || !c || !dh || !dz || !dc_prev || B <= 0 || H <= 0)
    return st::fail(ST_ERR_INVALID, "lstm_gate_bwd: bad arguments");
  lstm_gate_bwd_kernel<<<grid_for((long long)B * H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      act, c_prev, c, dh, dc_next, dz, dc_prev, B, H);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_wave_gate_fwd(const float* z, float* y, int B, int H, void* stream) {
  if (!z || !y || B <= 0 || H <= 0) return st::fail(ST_ERR_INVALID, "wave_gate_fwd: bad arguments");
  wave_gate_fwd_kernel<<<grid_for((long long)B * H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(z, y, B, H);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_wave_gate_bwd(const float* z, const float* dy, float* dz, int B, int H, void* stream) {
  if (!z || !dy || !dz || B <= 0 || H <= 0) return st::fail(ST_ERR_INVALID, "wave_gate_bwd: bad arguments");
  wave_gate_bwd_kernel<<<grid_for((long long)B * H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(z, dy, dz, B, H);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_sequence_last_step(const float* src, float* dst, int B, int steps, int dim, int scatter, void* stream) {
  if (!src || !dst || B <= 0 || steps <= 0 || dim <= 0) return st::fail(ST_ERR_INVALID, "sequence_last_step: bad arguments");
  last_step_kernel<<<grid_for((long long)B * dim), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(src, dst, B, steps, dim,
                                                                                                     scatter);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
