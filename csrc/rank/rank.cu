// Row-wise rank selection (top-k / bottom-k / mid-k) and row compaction.
//
// Selection semantics (crates/st-core/src/backend/rankk_software.rs:38-110, the CPU mirror of
// cuda_topk_rankk.cu): non-finite entries are ignored; candidates are ordered by value
// (descending for top, ascending for bottom and mid) with the LOWER column index winning ties;
// top/bottom take the first k, mid takes the k entries centred in the ascending order
// (start = (finite - take) / 2); unused output slots hold NaN / -1.
//
// One CTA sorts one row in shared memory with a bitonic network over 64-bit keys
// (order-preserving float bits in the high word, column index in the low word), which
// gives the exact, deterministic order in one pass for rows of up to 8192 columns.  k = 1 is a
// block arg-max/arg-min without sorting.  (The reference keeps 8 candidates per thread and lets
// thread 0 select serially.)
//
// Compaction (crates/st-kernel-contracts/src/compaction.rs:369-400): per row, keep the entries
// with low <= v <= high in their original order, write values and column indices densely,
// zero the padding and return the per-row counts.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace {
using namespace st;

enum Mode : int { TOP = 0, BOTTOM = 1, MID = 2 };

__device__ __forceinline__ unsigned orderable(float v) {
  unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending order of floats
}
__device__ __forceinline__ float from_orderable(unsigned o) {
  unsigned u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
  return __uint_as_float(u);
}

constexpr unsigned long long KEY_INVALID = 0xFFFFFFFFFFFFFFFFull;

__global__ void rank_select_kernel(const float* __restrict__ in, float* __restrict__ out_v,
                                   int* __restrict__ out_i, int rows, int cols, int k, int mode,
                                   int padded) {
  extern __shared__ unsigned long long keys[];
  __shared__ int s_finite;
  const int row = blockIdx.x;
  const float* x = in + (size_t)row * cols;
  if (threadIdx.x == 0) s_finite = 0;
  __syncthreads();
  int local = 0;
  for (int c = threadIdx.x; c < padded; c += blockDim.x) {
    unsigned long long key = KEY_INVALID;
    if (c < cols) {
      const float v = x[c];
      if (isfinite(v)) {
        unsigned o = orderable(v);
        if (mode == TOP) o = ~o;  // descending value == ascending key
        key = (static_cast<unsigned long long>(o) << 32) | static_cast<unsigned>(c);
        ++local;
      }
    }
    keys[c] = key;
  }
  atomicAdd(&s_finite, local);
  __syncthreads();
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < padded / 2; t += blockDim.x) {
        const int lo = (t / stride) * (stride << 1) + (t % stride);
        const int hi = lo + stride;
        const bool up = ((lo & size) == 0);
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  const int finite = s_finite;
  const int take = min(k, finite);
  const int start = (mode == MID) ? (finite - take) / 2 : 0;
  for (int s = threadIdx.x; s < k; s += blockDim.x) {
    float v = __int_as_float(0x7FC00000);
    int idx = -1;
    if (s < take) {
      const unsigned long long key = keys[start + s];
      unsigned o = static_cast<unsigned>(key >> 32);
      if (mode == TOP) o = ~o;
      v = from_orderable(o);
      idx = static_cast<int>(key & 0xFFFFFFFFu);
    }
    out_v[(size_t)row * k + s] = v;
    out_i[(size_t)row * k + s] = idx;
  }
}

// k == 1: block arg-max (mode TOP) / arg-min (BOTTOM); lower index wins ties.
__global__ void rank_k1_kernel(const float* __restrict__ in, float* __restrict__ out_v,
                               int* __restrict__ out_i, int rows, int cols, int mode) {
  __shared__ unsigned long long sh[32];
  const int row = blockIdx.x;
  const float* x = in + (size_t)row * cols;
  unsigned long long best = KEY_INVALID;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = x[c];
    if (!isfinite(v)) continue;
    unsigned o = orderable(v);
    if (mode == TOP) o = ~o;
    const unsigned long long key = (static_cast<unsigned long long>(o) << 32) | static_cast<unsigned>(c);
    best = key < best ? key : best;
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other < best ? other : best;
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = best;
  __syncthreads();
  if (w == 0) {
    best = l < (blockDim.x >> 5) ? sh[l] : KEY_INVALID;
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other < best ? other : best;
    }
    if (l == 0) {
      if (best == KEY_INVALID) {
        out_v[row] = __int_as_float(0x7FC00000);
        out_i[row] = -1;
      } else {
        unsigned o = static_cast<unsigned>(best >> 32);
        if (mode == TOP) o = ~o;
        out_v[row] = from_orderable(o);
        out_i[row] = static_cast<int>(best & 0xFFFFFFFFu);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
compact_rows_kernel(const float* __restrict__ in, float* __restrict__ out_v, int* __restrict__ out_i,
                    int* __restrict__ counts, int rows, int cols, float low, float high) {
  __shared__ int warp_tot[8];
  __shared__ int base;
  const int row = blockIdx.x;
  const float* x = in + (size_t)row * cols;
  float* ov = out_v + (size_t)row * cols;
  int* oi = out_i + (size_t)row * cols;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  for (int c0 = 0; c0 < cols; c0 += 256) {
    const int c = c0 + threadIdx.x;
    const float v = c < cols ? x[c] : 0.0f;
    const bool keep = c < cols && v >= low && v <= high;  // NaN fails both comparisons
    const unsigned ballot = __ballot_sync(0xffffffffu, keep);
    const int in_warp = __popc(ballot & ((1u << l) - 1u));
    if (l == 0) warp_tot[w] = __popc(ballot);
    __syncthreads();
    int before = base;
    for (int i = 0; i < w; ++i) before += warp_tot[i];
    if (keep) {
      ov[before + in_warp] = v;
      oi[before + in_warp] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int i = 0; i < 8; ++i) t += warp_tot[i];
      base += t;
    }
    __syncthreads();
  }
  const int n = base;
  for (int c = n + threadIdx.x; c < cols; c += 256) {
    ov[c] = 0.0f;
    oi[c] = 0;
  }
  if (threadIdx.x == 0) counts[row] = n;
}

// dst[r, p*k + s] = src_p[r, s] for every peer p: gathers the candidate lists of all ranks.
__global__ void gather_candidates_kernel(const float* const* __restrict__ vals, const int* const* __restrict__ idxs,
                                         float* __restrict__ dst_v, int* __restrict__ dst_i, int world,
                                         int rows, int k) {
  const long long total = (long long)world * rows * k;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int s = i % k;
    const long long t = i / k;
    const int r = t % rows;
    const int p = t / rows;
    dst_v[((long long)r * world + p) * k + s] = vals[p][(long long)r * k + s];
    dst_i[((long long)r * world + p) * k + s] = idxs[p][(long long)r * k + s];
  }
}

}  // namespace

// mode: 0 top, 1 bottom, 2 mid.  in: fp32 [rows, cols]; out_v fp32 [rows, k]; out_i int32 [rows, k].
ST_API int st_rank_select(const float* in, float* out_v, int* out_i, int rows, int cols, int k, int mode,
                          void* stream_v) {
  if (rows < 0 || cols < 0 || k < 0) return st::fail(ST_ERR_INVALID, "rank_select: negative dimension");
  if (rows == 0 || k == 0) return ST_OK;
  if (mode < 0 || mode > 2) return st::fail(ST_ERR_INVALID, "rank_select: mode must be 0 (top), 1 (bottom) or 2 (mid)");
  if (cols > 8192) return st::fail(ST_ERR_TOO_LARGE, "rank_select: rows of more than 8192 columns are not supported");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_v);
  if (k == 1 && mode != MID) {
    rank_k1_kernel<<<rows, cols >= 1024 ? 256 : 64, 0, s>>>(in, out_v, out_i, rows, cols, mode);
    ST_CUDA_CHECK(cudaGetLastError());
    return ST_OK;
  }
  int padded = 2;
  while (padded < cols) padded <<= 1;
  const size_t smem = (size_t)padded * sizeof(unsigned long long);
  static bool cfg = false;
  if (!cfg) {
    ST_CUDA_CHECK(cudaFuncSetAttribute(rank_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 8));
    cfg = true;
  }
  int threads = padded / 2;
  threads = threads < 32 ? 32 : (threads > 1024 ? 1024 : threads);
  rank_select_kernel<<<rows, threads, smem, s>>>(in, out_v, out_i, rows, cols, k, mode, padded);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

ST_API int st_compact_rows(const float* in, float* out_v, int* out_i, int* counts, int rows, int cols,
                           float low, float high, void* stream_v) {
  if (rows < 0 || cols < 0) return st::fail(ST_ERR_INVALID, "compaction dimensions must be non-negative");
  if (!(low <= high) || isinf(low) || isinf(high))
    return st::fail(ST_ERR_INVALID, "compaction bounds must be finite and ordered");
  if (rows == 0) return ST_OK;
  compact_rows_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(in, out_v, out_i, counts,
                                                                                 rows, cols, low, high);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

// vals / idxs: device arrays of `world` pointers (peer memory allowed) to [rows, k] candidate lists.
ST_API int st_gather_candidates(const void* vals, const void* idxs, float* dst_v, int* dst_i, int world,
                                int rows, int k, void* stream_v) {
  const long long total = (long long)world * rows * k;
  if (total <= 0) return ST_OK;
  long long blocks = (total + 255) / 256;
  if (blocks > 1024) blocks = 1024;
  gather_candidates_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const float* const*>(vals), static_cast<const int* const*>(idxs), dst_v, dst_i, world, rows, k);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}
