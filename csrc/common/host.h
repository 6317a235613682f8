// Host-side helpers shared by the launchers: error reporting, the per-process error word
// that bounded device waits write to, TMA tensor-map encoding and device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ST_API extern "C" __attribute__((visibility("default")))

// Return codes of every launcher in this library.
enum StStatus : int {
  ST_OK = 0,
  ST_ERR_INVALID = 1,    // bad argument (shape / alignment / unsupported combination)
  ST_ERR_CUDA = 2,       // CUDA runtime or driver error; see st_last_error()
  ST_ERR_TOO_LARGE = 3,  // exceeds a fixed capacity
  ST_ERR_DEVICE = 4,     // a device-side bounded wait or bounds check reported failure
};

namespace st {

// Records `msg` for st_last_error() and returns `code`.
int fail(int code, const char* msg);
int fail_cuda(cudaError_t e, const char* where);

// Device pointer of the 4-word error record (mapped pinned host memory) for the current
// device.  Kernels receive it as an argument.
unsigned* error_word();

int sm_count();

// Index of the current CUDA device clamped to [0, kMaxDevices): per-device launcher state (shared-memory
// opt-in flags, cached addresses) is keyed by it, because function attributes are set per device.
constexpr int kMaxDevices = 16;
int current_device();

// Encodes a tiled bf16/fp32 tensor map.  dims/strides innermost first; strides in bytes for
// dims 1..rank-1.  Returns false (after recording the error) on failure.
bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                 CUtensorMapSwizzle swizzle);

bool encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                         uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

}  // namespace st

#define ST_CUDA_CHECK(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return st::fail_cuda(_e, #expr);   \
  } while (0)
