// Tensor-level C ABI: opaque 2-D float tensors and a runtime handle, for callers that bind through a C header
// (Go, Julia, C, COBOL shims) instead of Python.  Same function names and calling conventions as the
// reference's spiraltorch-sys crate (bindings/spiraltorch-sys/src/lib.rs:130-1640): every function that can fail
// returns null / false / 0 and leaves a message for spiraltorch_last_error_message; success clears it.
//
// Tensors here are host tensors: the arithmetic runs on the CPU (row-blocked loops; the runtime variants split
// the rows of the result over the runtime's worker threads).  The GPU backends of the reference's enum are
// refused by name - device kernels are reached through the launchers of the CUDA library, which take raw device
// pointers and a stream.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#define ST_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;
void set_error(const std::string& m) { g_error = m; }
void clear_error() { g_error.clear(); }

struct SpiralTensor {
  size_t rows = 0, cols = 0;
  std::vector<float> data;
};

struct RuntimeHandle {
  size_t workers = 1;
  std::string name;
};

SpiralTensor* make(size_t rows, size_t cols) {
  if (rows == 0 || cols == 0) {
    set_error("tensor dimensions must be positive");
    return nullptr;
  }
  if (rows > SIZE_MAX / cols / sizeof(float)) {
    set_error("tensor dimensions overflow");
    return nullptr;
  }
  auto* t = new (std::nothrow) SpiralTensor;
  if (!t) {
    set_error("out of memory");
    return nullptr;
  }
  t->rows = rows;
  t->cols = cols;
  try {
    t->data.assign(rows * cols, 0.0f);
  } catch (...) {
    delete t;
    set_error("out of memory");
    return nullptr;
  }
  return t;
}

const SpiralTensor* need(const SpiralTensor* t, const char* what) {
  if (!t) set_error(std::string(what) + " received a null tensor handle");
  return t;
}

// Runs fn(row_begin, row_end) over [0, rows) on up to `workers` threads.
void parallel_rows(size_t rows, size_t workers, const std::function<void(size_t, size_t)>& fn) {
  workers = std::max<size_t>(1, std::min(workers, rows));
  if (workers == 1) {
    fn(0, rows);
    return;
  }
  std::vector<std::thread> th;
  const size_t per = (rows + workers - 1) / workers;
  for (size_t w = 0; w < workers; ++w) {
    const size_t lo = w * per, hi = std::min(rows, lo + per);
    if (lo >= hi) break;
    th.emplace_back([&fn, lo, hi] { fn(lo, hi); });
  }
  for (auto& t : th) t.join();
}

enum Epilogue { EP_NONE = 0, EP_BIAS_RELU = 1, EP_BIAS_GELU = 2, EP_BIAS_ADD_RELU = 3 };

float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.0f + std::tanh(k * (x + 0.044715f * x * x * x)));
}

SpiralTensor* matmul_impl(const SpiralTensor* a, const SpiralTensor* b, int backend, Epilogue ep, const float* bias,
                          size_t bias_len, const SpiralTensor* residual, size_t workers, const char* what) {
  if (!need(a, what) || !need(b, what)) return nullptr;
  if (backend < 0 || backend > 5) {
    set_error(std::string(what) + ": unknown matmul backend");
    return nullptr;
  }
  if (backend >= 4) {
    set_error(std::string(what) + ": GPU matmul backends are not part of the host tensor ABI; use the device launchers");
    return nullptr;
  }
  if (a->cols != b->rows) {
    set_error(std::string(what) + ": inner dimensions differ (" + std::to_string(a->rows) + "x" + std::to_string(a->cols) +
              " times " + std::to_string(b->rows) + "x" + std::to_string(b->cols) + ")");
    return nullptr;
  }
  if (ep != EP_NONE) {
    if (!bias) {
      set_error(std::string(what) + " received a null bias pointer");
      return nullptr;
    }
    if (bias_len != b->cols) {
      set_error(std::string(what) + ": bias length " + std::to_string(bias_len) + " does not match " + std::to_string(b->cols) + " columns");
      return nullptr;
    }
  }
  if (ep == EP_BIAS_ADD_RELU) {
    if (!need(residual, what)) return nullptr;
    if (residual->rows != a->rows || residual->cols != b->cols) {
      set_error(std::string(what) + ": residual shape does not match the product");
      return nullptr;
    }
  }
  SpiralTensor* c = make(a->rows, b->cols);
  if (!c) return nullptr;
  const size_t K = a->cols, N = b->cols;
  parallel_rows(a->rows, workers, [&](size_t lo, size_t hi) {
    for (size_t i = lo; i < hi; ++i) {
      float* cr = c->data.data() + i * N;
      const float* ar = a->data.data() + i * K;
      for (size_t k = 0; k < K; ++k) {           // row of A times rows of B: unit-stride inner loop
        const float av = ar[k];
        const float* br = b->data.data() + k * N;
        for (size_t j = 0; j < N; ++j) cr[j] += av * br[j];
      }
      if (ep != EP_NONE) {
        for (size_t j = 0; j < N; ++j) {
          float v = cr[j] + bias[j];
          if (ep == EP_BIAS_ADD_RELU) v += residual->data[i * N + j];
          cr[j] = ep == EP_BIAS_GELU ? gelu_tanh(v) : std::max(v, 0.0f);
        }
      }
    }
  });
  clear_error();
  return c;
}

SpiralTensor* binary_impl(const SpiralTensor* a, const SpiralTensor* b, int op, size_t workers, const char* what) {
  if (!need(a, what) || !need(b, what)) return nullptr;
  if (a->rows != b->rows || a->cols != b->cols) {
    set_error(std::string(what) + ": shape mismatch");
    return nullptr;
  }
  SpiralTensor* c = make(a->rows, a->cols);
  if (!c) return nullptr;
  parallel_rows(a->rows, workers, [&](size_t lo, size_t hi) {
    for (size_t i = lo * a->cols; i < hi * a->cols; ++i)
      c->data[i] = op == 0 ? a->data[i] + b->data[i] : (op == 1 ? a->data[i] - b->data[i] : a->data[i] * b->data[i]);
  });
  clear_error();
  return c;
}

SpiralTensor* scale_impl(const SpiralTensor* a, float s, const char* what) {
  if (!need(a, what)) return nullptr;
  SpiralTensor* c = make(a->rows, a->cols);
  if (!c) return nullptr;
  for (size_t i = 0; i < a->data.size(); ++i) c->data[i] = a->data[i] * s;
  clear_error();
  return c;
}

SpiralTensor* transpose_impl(const SpiralTensor* a, const char* what) {
  if (!need(a, what)) return nullptr;
  SpiralTensor* c = make(a->cols, a->rows);
  if (!c) return nullptr;
  for (size_t i = 0; i < a->rows; ++i)
    for (size_t j = 0; j < a->cols; ++j) c->data[j * a->rows + i] = a->data[i * a->cols + j];
  clear_error();
  return c;
}

SpiralTensor* reshape_impl(const SpiralTensor* a, size_t rows, size_t cols, const char* what) {
  if (!need(a, what)) return nullptr;
  if (rows == 0 || cols == 0 || rows * cols != a->data.size()) {
    set_error(std::string(what) + ": cannot reshape " + std::to_string(a->rows) + "x" + std::to_string(a->cols) + " to " +
              std::to_string(rows) + "x" + std::to_string(cols));
    return nullptr;
  }
  SpiralTensor* c = make(rows, cols);
  if (!c) return nullptr;
  c->data = a->data;
  clear_error();
  return c;
}

SpiralTensor* softmax_impl(const SpiralTensor* a, size_t workers, const char* what) {
  if (!need(a, what)) return nullptr;
  SpiralTensor* c = make(a->rows, a->cols);
  if (!c) return nullptr;
  parallel_rows(a->rows, workers, [&](size_t lo, size_t hi) {
    for (size_t i = lo; i < hi; ++i) {
      const float* x = a->data.data() + i * a->cols;
      float* y = c->data.data() + i * a->cols;
      float m = x[0];
      for (size_t j = 1; j < a->cols; ++j) m = std::max(m, x[j]);
      double s = 0.0;
      for (size_t j = 0; j < a->cols; ++j) s += (y[j] = std::exp(x[j] - m));
      const float inv = (float)(1.0 / s);
      for (size_t j = 0; j < a->cols; ++j) y[j] *= inv;
    }
  });
  clear_error();
  return c;
}

SpiralTensor* random_impl(size_t rows, size_t cols, bool normal, float p0, float p1, uint64_t seed, bool has_seed,
                          const char* what) {
  if (normal ? !(p1 >= 0.0f && std::isfinite(p0) && std::isfinite(p1)) : !(p0 < p1 && std::isfinite(p0) && std::isfinite(p1))) {
    set_error(std::string(what) + (normal ? ": std must be finite and non-negative" : ": min must be finite and below max"));
    return nullptr;
  }
  SpiralTensor* c = make(rows, cols);
  if (!c) return nullptr;
  std::mt19937_64 rng(has_seed ? seed : std::random_device{}());
  if (normal) {
    std::normal_distribution<float> d(p0, p1 > 0.0f ? p1 : 1.0f);
    for (auto& v : c->data) v = p1 > 0.0f ? d(rng) : p0;
  } else {
    std::uniform_real_distribution<float> d(p0, p1);
    for (auto& v : c->data) v = d(rng);
  }
  clear_error();
  return c;
}

size_t workers_of(const RuntimeHandle* rt, const char* what, bool* ok) {
  if (!rt) {
    set_error(std::string(what) + " received a null runtime handle");
    *ok = false;
    return 1;
  }
  *ok = true;
  return rt->workers;
}

// ---- DLPack (CPU, float32, 2-D) ----------------------------------------------------------------------------
struct DLDevice { int32_t device_type; int32_t device_id; };
struct DLDataType { uint8_t code; uint8_t bits; uint16_t lanes; };
struct DLTensor {
  void* data; DLDevice device; int32_t ndim; DLDataType dtype; int64_t* shape; int64_t* strides; uint64_t byte_offset;
};
struct DLManagedTensor {
  DLTensor dl_tensor; void* manager_ctx; void (*deleter)(DLManagedTensor*);
};
struct Exported {
  std::vector<float> data;
  int64_t shape[2];
  int64_t strides[2];
};
void dl_deleter(DLManagedTensor* m) {
  if (!m) return;
  delete static_cast<Exported*>(m->manager_ctx);
  delete m;
}

}  // namespace

struct StRoundtableSummary {
  size_t above, here, beneath;
  float energy_above, energy_here, energy_beneath;
};

ST_HOST_API const char* spiraltorch_version() { return "spiraltorch-b200 0.2.0 (host tensor ABI 1)"; }
ST_HOST_API size_t spiraltorch_last_error_length() { return g_error.size(); }
// Copies the message (NUL-terminated, truncated to capacity - 1); returns the bytes written without the NUL.
ST_HOST_API size_t spiraltorch_last_error_message(char* buffer, size_t capacity) {
  if (!buffer || capacity == 0) return 0;
  const size_t n = std::min(capacity - 1, g_error.size());
  memcpy(buffer, g_error.data(), n);
  buffer[n] = 0;
  return n;
}
ST_HOST_API void spiraltorch_clear_last_error() { clear_error(); }

ST_HOST_API SpiralTensor* spiraltorch_tensor_zeros(size_t rows, size_t cols) {
  SpiralTensor* t = make(rows, cols);
  if (t) clear_error();
  return t;
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_from_dense(size_t rows, size_t cols, const float* data, size_t len) {
  if (!data) {
    set_error("tensor_from_dense received a null data pointer");
    return nullptr;
  }
  if (rows == 0 || cols == 0 || len != rows * cols) {
    set_error("tensor_from_dense: data length " + std::to_string(len) + " does not match " + std::to_string(rows) + "x" + std::to_string(cols));
    return nullptr;
  }
  SpiralTensor* t = make(rows, cols);
  if (!t) return nullptr;
  memcpy(t->data.data(), data, len * sizeof(float));
  clear_error();
  return t;
}
ST_HOST_API void spiraltorch_tensor_free(SpiralTensor* t) { delete t; }
ST_HOST_API bool spiraltorch_tensor_shape(const SpiralTensor* t, size_t* rows_out, size_t* cols_out) {
  if (!need(t, "tensor_shape")) return false;
  if (!rows_out || !cols_out) {
    set_error("tensor_shape received a null output pointer");
    return false;
  }
  *rows_out = t->rows;
  *cols_out = t->cols;
  clear_error();
  return true;
}
ST_HOST_API size_t spiraltorch_tensor_elements(const SpiralTensor* t) {
  if (!need(t, "tensor_elements")) return 0;
  clear_error();
  return t->data.size();
}
ST_HOST_API bool spiraltorch_tensor_copy_data(const SpiralTensor* t, float* out, size_t len) {
  if (!need(t, "tensor_copy_data")) return false;
  if (!out || len < t->data.size()) {
    set_error("tensor_copy_data: output buffer is null or too small (" + std::to_string(len) + " < " + std::to_string(t->data.size()) + ")");
    return false;
  }
  memcpy(out, t->data.data(), t->data.size() * sizeof(float));
  clear_error();
  return true;
}
ST_HOST_API bool spiraltorch_tensor_copy_row(const SpiralTensor* t, size_t index, float* out, size_t len) {
  if (!need(t, "tensor_copy_row")) return false;
  if (index >= t->rows || !out || len < t->cols) {
    set_error("tensor_copy_row: row index out of range or output buffer too small");
    return false;
  }
  memcpy(out, t->data.data() + index * t->cols, t->cols * sizeof(float));
  clear_error();
  return true;
}
ST_HOST_API bool spiraltorch_tensor_copy_column(const SpiralTensor* t, size_t index, float* out, size_t len) {
  if (!need(t, "tensor_copy_column")) return false;
  if (index >= t->cols || !out || len < t->rows) {
    set_error("tensor_copy_column: column index out of range or output buffer too small");
    return false;
  }
  for (size_t i = 0; i < t->rows; ++i) out[i] = t->data[i * t->cols + index];
  clear_error();
  return true;
}

ST_HOST_API void* spiraltorch_tensor_to_dlpack(const SpiralTensor* t) {
  if (!need(t, "tensor_to_dlpack")) return nullptr;
  auto* ex = new Exported;
  ex->data = t->data;                       // the capsule owns a copy: the tensor handle stays valid on its own
  ex->shape[0] = (int64_t)t->rows; ex->shape[1] = (int64_t)t->cols;
  ex->strides[0] = (int64_t)t->cols; ex->strides[1] = 1;
  auto* m = new DLManagedTensor;
  m->dl_tensor.data = ex->data.data();
  m->dl_tensor.device = {1 /* kDLCPU */, 0};
  m->dl_tensor.ndim = 2;
  m->dl_tensor.dtype = {2 /* kDLFloat */, 32, 1};
  m->dl_tensor.shape = ex->shape;
  m->dl_tensor.strides = ex->strides;
  m->dl_tensor.byte_offset = 0;
  m->manager_ctx = ex;
  m->deleter = dl_deleter;
  clear_error();
  return m;
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_from_dlpack(void* managed) {
  auto* m = static_cast<DLManagedTensor*>(managed);
  if (!m) {
    set_error("tensor_from_dlpack received a null capsule");
    return nullptr;
  }
  const DLTensor& d = m->dl_tensor;
  if (d.device.device_type != 1 || d.ndim != 2 || d.dtype.code != 2 || d.dtype.bits != 32 || d.dtype.lanes != 1 || !d.data) {
    set_error("tensor_from_dlpack: only 2-D float32 CPU tensors are accepted");
    return nullptr;
  }
  const size_t rows = (size_t)d.shape[0], cols = (size_t)d.shape[1];
  const int64_t s0 = d.strides ? d.strides[0] : (int64_t)cols, s1 = d.strides ? d.strides[1] : 1;
  SpiralTensor* t = make(rows, cols);
  if (!t) return nullptr;
  const float* src = reinterpret_cast<const float*>(static_cast<const char*>(d.data) + d.byte_offset);
  for (size_t i = 0; i < rows; ++i)
    for (size_t j = 0; j < cols; ++j) t->data[i * cols + j] = src[(int64_t)i * s0 + (int64_t)j * s1];
  if (m->deleter) m->deleter(m);            // the data was copied: the producer's capsule is consumed
  clear_error();
  return t;
}
ST_HOST_API void spiraltorch_dlpack_drop_exported_state(void* managed) { dl_deleter(static_cast<DLManagedTensor*>(managed)); }

ST_HOST_API SpiralTensor* spiraltorch_tensor_add(const SpiralTensor* a, const SpiralTensor* b) { return binary_impl(a, b, 0, 1, "tensor_add"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_sub(const SpiralTensor* a, const SpiralTensor* b) { return binary_impl(a, b, 1, 1, "tensor_sub"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_hadamard(const SpiralTensor* a, const SpiralTensor* b) { return binary_impl(a, b, 2, 1, "tensor_hadamard"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_scale(const SpiralTensor* a, float s) { return scale_impl(a, s, "tensor_scale"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_transpose(const SpiralTensor* a) { return transpose_impl(a, "tensor_transpose"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_reshape(const SpiralTensor* a, size_t rows, size_t cols) { return reshape_impl(a, rows, cols, "tensor_reshape"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_row_softmax(const SpiralTensor* a, int /*backend*/) { return softmax_impl(a, 1, "tensor_row_softmax"); }
ST_HOST_API SpiralTensor* spiraltorch_tensor_random_uniform(size_t rows, size_t cols, float min, float max, uint64_t seed, bool has_seed) {
  return random_impl(rows, cols, false, min, max, seed, has_seed, "tensor_random_uniform");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_random_normal(size_t rows, size_t cols, float mean, float std, uint64_t seed, bool has_seed) {
  return random_impl(rows, cols, true, mean, std, seed, has_seed, "tensor_random_normal");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul(const SpiralTensor* a, const SpiralTensor* b) {
  return matmul_impl(a, b, 0, EP_NONE, nullptr, 0, nullptr, 1, "tensor_matmul");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_with_backend(const SpiralTensor* a, const SpiralTensor* b, int backend) {
  return matmul_impl(a, b, backend, EP_NONE, nullptr, 0, nullptr, 1, "tensor_matmul_with_backend");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_bias_relu(const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n) {
  return matmul_impl(a, b, 0, EP_BIAS_RELU, bias, n, nullptr, 1, "tensor_matmul_bias_relu");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_bias_relu_with_backend(const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, int backend) {
  return matmul_impl(a, b, backend, EP_BIAS_RELU, bias, n, nullptr, 1, "tensor_matmul_bias_relu_with_backend");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_bias_gelu(const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n) {
  return matmul_impl(a, b, 0, EP_BIAS_GELU, bias, n, nullptr, 1, "tensor_matmul_bias_gelu");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_bias_gelu_with_backend(const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, int backend) {
  return matmul_impl(a, b, backend, EP_BIAS_GELU, bias, n, nullptr, 1, "tensor_matmul_bias_gelu_with_backend");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_bias_add_relu(const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, const SpiralTensor* residual) {
  return matmul_impl(a, b, 0, EP_BIAS_ADD_RELU, bias, n, residual, 1, "tensor_matmul_bias_add_relu");
}
ST_HOST_API SpiralTensor* spiraltorch_tensor_matmul_bias_add_relu_with_backend(const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, const SpiralTensor* residual, int backend) {
  return matmul_impl(a, b, backend, EP_BIAS_ADD_RELU, bias, n, residual, 1, "tensor_matmul_bias_add_relu_with_backend");
}

// ---- runtime handle: the same operations with their rows split over worker threads ----------------------------
ST_HOST_API RuntimeHandle* spiraltorch_runtime_new(size_t worker_threads, const char* thread_name) {
  auto* rt = new (std::nothrow) RuntimeHandle;
  if (!rt) {
    set_error("out of memory");
    return nullptr;
  }
  const size_t hw = std::max(1u, std::thread::hardware_concurrency());
  rt->workers = worker_threads == 0 ? hw : std::min<size_t>(worker_threads, 256);
  rt->name = thread_name ? thread_name : "spiraltorch-runtime";
  clear_error();
  return rt;
}
ST_HOST_API void spiraltorch_runtime_free(RuntimeHandle* rt) { delete rt; }
ST_HOST_API size_t spiraltorch_runtime_worker_count(const RuntimeHandle* rt) {
  bool ok;
  const size_t w = workers_of(rt, "runtime_worker_count", &ok);
  if (!ok) return 0;
  clear_error();
  return w;
}
#define RT_WORKERS(what)                         \
  bool ok_;                                      \
  const size_t w_ = workers_of(rt, what, &ok_);  \
  if (!ok_) return nullptr;
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_add(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b) { RT_WORKERS("runtime_tensor_add") return binary_impl(a, b, 0, w_, "runtime_tensor_add"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_sub(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b) { RT_WORKERS("runtime_tensor_sub") return binary_impl(a, b, 1, w_, "runtime_tensor_sub"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_hadamard(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b) { RT_WORKERS("runtime_tensor_hadamard") return binary_impl(a, b, 2, w_, "runtime_tensor_hadamard"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_scale(const RuntimeHandle* rt, const SpiralTensor* a, float s) { RT_WORKERS("runtime_tensor_scale") (void)w_; return scale_impl(a, s, "runtime_tensor_scale"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_transpose(const RuntimeHandle* rt, const SpiralTensor* a) { RT_WORKERS("runtime_tensor_transpose") (void)w_; return transpose_impl(a, "runtime_tensor_transpose"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_reshape(const RuntimeHandle* rt, const SpiralTensor* a, size_t rows, size_t cols) { RT_WORKERS("runtime_tensor_reshape") (void)w_; return reshape_impl(a, rows, cols, "runtime_tensor_reshape"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_row_softmax(const RuntimeHandle* rt, const SpiralTensor* a, int /*backend*/) { RT_WORKERS("runtime_tensor_row_softmax") return softmax_impl(a, w_, "runtime_tensor_row_softmax"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_random_uniform(const RuntimeHandle* rt, size_t rows, size_t cols, float min, float max, uint64_t seed, bool has_seed) { RT_WORKERS("runtime_tensor_random_uniform") (void)w_; return random_impl(rows, cols, false, min, max, seed, has_seed, "runtime_tensor_random_uniform"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_random_normal(const RuntimeHandle* rt, size_t rows, size_t cols, float mean, float std, uint64_t seed, bool has_seed) { RT_WORKERS("runtime_tensor_random_normal") (void)w_; return random_impl(rows, cols, true, mean, std, seed, has_seed, "runtime_tensor_random_normal"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b) { RT_WORKERS("runtime_tensor_matmul") return matmul_impl(a, b, 0, EP_NONE, nullptr, 0, nullptr, w_, "runtime_tensor_matmul"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_with_backend(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, int backend) { RT_WORKERS("runtime_tensor_matmul_with_backend") return matmul_impl(a, b, backend, EP_NONE, nullptr, 0, nullptr, w_, "runtime_tensor_matmul_with_backend"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_bias_relu(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n) { RT_WORKERS("runtime_tensor_matmul_bias_relu") return matmul_impl(a, b, 0, EP_BIAS_RELU, bias, n, nullptr, w_, "runtime_tensor_matmul_bias_relu"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_bias_relu_with_backend(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, int backend) { RT_WORKERS("runtime_tensor_matmul_bias_relu_with_backend") return matmul_impl(a, b, backend, EP_BIAS_RELU, bias, n, nullptr, w_, "runtime_tensor_matmul_bias_relu_with_backend"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_bias_gelu(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n) { RT_WORKERS("runtime_tensor_matmul_bias_gelu") return matmul_impl(a, b, 0, EP_BIAS_GELU, bias, n, nullptr, w_, "runtime_tensor_matmul_bias_gelu"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_bias_gelu_with_backend(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, int backend) { RT_WORKERS("runtime_tensor_matmul_bias_gelu_with_backend") return matmul_impl(a, b, backend, EP_BIAS_GELU, bias, n, nullptr, w_, "runtime_tensor_matmul_bias_gelu_with_backend"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_bias_add_relu(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, const SpiralTensor* residual) { RT_WORKERS("runtime_tensor_matmul_bias_add_relu") return matmul_impl(a, b, 0, EP_BIAS_ADD_RELU, bias, n, residual, w_, "runtime_tensor_matmul_bias_add_relu"); }
ST_HOST_API SpiralTensor* spiraltorch_runtime_tensor_matmul_bias_add_relu_with_backend(const RuntimeHandle* rt, const SpiralTensor* a, const SpiralTensor* b, const float* bias, size_t n, const SpiralTensor* residual, int backend) { RT_WORKERS("runtime_tensor_matmul_bias_add_relu_with_backend") return matmul_impl(a, b, backend, EP_BIAS_ADD_RELU, bias, n, residual, w_, "runtime_tensor_matmul_bias_add_relu_with_backend"); }

// Splits a gradient into the Above (0) / Here (1) / Beneath (2) bands of the roundtable by magnitude rank: the
// `above_k` largest magnitudes go Above, the `beneath_k` smallest of the rest Beneath, everything at or below
// `tolerance` back to Here (bindings/spiraltorch-sys/src/lib.rs:1518-1620).
ST_HOST_API bool spiraltorch_roundtable_classify(const float* gradient, size_t len, size_t above_k, size_t here_k,
                                                 size_t beneath_k, float tolerance, uint8_t* assignments,
                                                 StRoundtableSummary* summary) {
  (void)here_k;   // the middle band is whatever the other two leave
  if (!gradient) { set_error("roundtable_classify received null gradient pointer"); return false; }
  if (len == 0) { set_error("roundtable_classify requires a non-empty gradient"); return false; }
  if (!assignments) { set_error("roundtable_classify assignments received a null pointer"); return false; }
  if (!summary) { set_error("roundtable_classify summary received a null pointer"); return false; }
  std::vector<size_t> order(len);
  for (size_t i = 0; i < len; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](size_t l, size_t r) { return std::fabs(gradient[l]) > std::fabs(gradient[r]); });
  std::vector<uint8_t> bands(len, 1);
  const size_t top = std::min(above_k, len);
  for (size_t i = 0; i < top; ++i) bands[order[i]] = 0;
  const size_t bottom = std::min(beneath_k, len - top);
  for (size_t i = 0; i < bottom; ++i) bands[order[len - 1 - i]] = 2;
  const float tol = std::max(tolerance, 0.0f);
  for (size_t i = 0; i < len; ++i)
    if (std::fabs(gradient[i]) <= tol) bands[i] = 1;
  memcpy(assignments, bands.data(), len);
  StRoundtableSummary s{0, 0, 0, 0.0f, 0.0f, 0.0f};
  for (size_t i = 0; i < len; ++i) {
    const float mag = std::isfinite(gradient[i]) ? std::fabs(gradient[i]) : 0.0f;
    if (bands[i] == 0) { ++s.above; s.energy_above += mag; }
    else if (bands[i] == 1) { ++s.here; s.energy_here += mag; }
    else { ++s.beneath; s.energy_beneath += mag; }
  }
  *summary = s;
  clear_error();
  return true;
}
