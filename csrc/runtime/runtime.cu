// Process-wide runtime state of the native library: last error string, the device error
// word written by bounded waits, tensor-map encoding through the driver entry point and
// cached device properties.
#include "../common/host.h"
#include "../common/ptx.cuh"

#include <mutex>
#include <string>
#include <cstdio>
#include <cstring>

namespace {
std::mutex g_mu;
std::string g_last_error;

using st::kMaxDevices;
unsigned* g_err_host[kMaxDevices] = {nullptr};
unsigned* g_err_dev[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    g_last_error = "cuTensorMapEncodeTiled entry point unavailable";
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

namespace {
// Setters of the per-translation-unit wait-limit words (registered by static initialisers, so the
// list itself must not depend on another static's construction order: plain array + counter).
constexpr int kMaxSetters = 64;
st::WaitLimitSetter g_setters[kMaxSetters];
int g_n_setters = 0;
}  // namespace

namespace st {

void register_wait_limit_setter(WaitLimitSetter fn) {
  if (g_n_setters < kMaxSetters) g_setters[g_n_setters++] = fn;
}

int fail(int code, const char* msg) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_last_error = msg ? msg : "";
  return code;
}

int fail_cuda(cudaError_t e, const char* where) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_last_error = std::string(where ? where : "") + ": " + cudaGetErrorString(e);
  return ST_ERR_CUDA;
}

unsigned* error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_err_dev[dev]) return g_err_dev[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_err_dev[dev]) return g_err_dev[dev];
  unsigned* h = nullptr;
  if (cudaHostAlloc(reinterpret_cast<void**>(&h), 4 * sizeof(unsigned), cudaHostAllocMapped) !=
      cudaSuccess)
    return nullptr;
  memset(h, 0, 4 * sizeof(unsigned));
  unsigned* d = nullptr;
  if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0) != cudaSuccess) return nullptr;
  g_err_host[dev] = h;
  g_err_dev[dev] = d;
  return d;
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  return dev;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                 CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return false;
  // The driver entry point needs a current context on the calling thread.  Threads that
  // have only used the runtime API lazily (e.g. an autograd worker) may not have one yet:
  // a no-op runtime call binds the primary context of the current device.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr,
                  bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf),
             "cuTensorMapEncodeTiled failed (%d): rank=%d base=%p dims=[%llu,%llu] stride0=%llu "
             "box=[%u,%u]",
             static_cast<int>(r), rank, base, (unsigned long long)dims[0],
             (unsigned long long)(rank > 1 ? dims[1] : 0),
             (unsigned long long)(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0);
    fail(ST_ERR_CUDA, buf);
    return false;
  }
  return true;
}

bool encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                         uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                         CUtensorMapSwizzle swizzle) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {row_stride_bytes};
  uint32_t box[2] = {box_inner, box_outer};
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, swizzle);
}

}  // namespace st

ST_API const char* st_last_error() {
  static thread_local std::string copy;
  std::lock_guard<std::mutex> lk(g_mu);
  copy = g_last_error;
  return copy.c_str();
}

// Copies the 4-word device error record of the current device into `out` and, when `clear`
// is non-zero, resets it.  Returns the error code (0 = none).  Needs no device sync: the
// record is in mapped host memory.
ST_API int st_read_error_word(unsigned* out, int clear) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  unsigned* h = g_err_host[dev];
  if (!h) {
    if (out) memset(out, 0, 4 * sizeof(unsigned));
    return 0;
  }
  unsigned code = reinterpret_cast<volatile unsigned*>(h)[0];
  if (out)
    for (int i = 0; i < 4; ++i) out[i] = reinterpret_cast<volatile unsigned*>(h)[i];
  if (clear) memset(h, 0, 4 * sizeof(unsigned));
  return static_cast<int>(code);
}

// Sets the limit of every bounded device-side wait (mbarrier, peer flag) on the CURRENT device, in
// nanoseconds; 0 restores the 2 s default.  Takes effect for kernels launched afterwards.
ST_API int st_set_wait_timeout_ns(unsigned long long ns) {
  if (ns == 0) ns = ST_WAIT_TIMEOUT_NS;
  for (int i = 0; i < g_n_setters; ++i) {
    cudaError_t e = g_setters[i](ns);
    if (e != cudaSuccess) return st::fail_cuda(e, "st_set_wait_timeout_ns");
  }
  return ST_OK;
}

ST_API int st_sm_count() { return st::sm_count(); }

ST_API int st_abi_version() { return 1; }
