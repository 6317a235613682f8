// JavaScript wrapper over the tensor-level C ABI, for a WebAssembly build of the host library
// (csrc/host/tensor_abi.cpp compiled with Emscripten, see build.sh).  Same surface as the Go and Julia
// packages: Tensor (dense row-major f32 matrices), fused matmul epilogues, seeded random fills, the
// roundtable classifier, version and last-error access.  The reference ships its browser binding as a
// wasm-bindgen crate (bindings/st-wasm/src/lib.rs); this one goes through the C ABI instead, so the
// exported names are the ones in include/spiraltorch_b200.h.
//
//   import createModule from "./spiraltorch_host.mjs";      // produced by build.sh
//   import { bind } from "./spiraltorch.mjs";
//   const st = bind(await createModule());
//   const y = st.Tensor.fromDense(2, 2, [1, 2, 3, 4]).matmul(st.Tensor.fromDense(2, 2, [0, 1, 1, 0]));
//   console.log(y.shape(), y.data()); y.free();

export function bind(M) {
  const registry = typeof FinalizationRegistry === "undefined" ? null
    : new FinalizationRegistry((ptr) => { M._spiraltorch_tensor_free(ptr); });

  function lastError() {
    const n = M._spiraltorch_last_error_length();
    if (n === 0) return "";
    const buf = M._malloc(n + 1);
    try {
      M._spiraltorch_last_error_message(buf, n + 1);
      return M.UTF8ToString(buf);
    } finally {
      M._free(buf);
    }
  }

  function check(ptr, what) {
    if (ptr === 0) {
      const msg = lastError();
      M._spiraltorch_clear_last_error();
      throw new Error(`spiraltorch: ${what} failed: ${msg || "unknown error"}`);
    }
    return ptr;
  }

  function withFloats(values, fn) {
    const arr = values instanceof Float32Array ? values : Float32Array.from(values);
    const buf = M._malloc(Math.max(arr.length, 1) * 4);
    try {
      M.HEAPF32.set(arr, buf >> 2);
      return fn(buf, arr.length);
    } finally {
      M._free(buf);
    }
  }

  class Tensor {
    constructor(ptr) {
      this.ptr = ptr;
      if (registry) registry.register(this, ptr, this);
    }

    static fromDense(rows, cols, values) {
      return withFloats(values, (buf, n) => new Tensor(check(M._spiraltorch_tensor_from_dense(rows, cols, buf, n), "from_dense")));
    }

    static zeros(rows, cols) {
      return new Tensor(check(M._spiraltorch_tensor_zeros(rows, cols), "zeros"));
    }

    // seed: a BigInt (the build uses -sWASM_BIGINT), or null / undefined for an unseeded fill
    static randomUniform(rows, cols, min, max, seed = null) {
      return new Tensor(check(M._spiraltorch_tensor_random_uniform(rows, cols, min, max, BigInt(seed ?? 0), seed != null), "random_uniform"));
    }

    static randomNormal(rows, cols, mean, std, seed = null) {
      return new Tensor(check(M._spiraltorch_tensor_random_normal(rows, cols, mean, std, BigInt(seed ?? 0), seed != null), "random_normal"));
    }

    free() {
      if (this.ptr !== 0) {
        if (registry) registry.unregister(this);
        M._spiraltorch_tensor_free(this.ptr);
        this.ptr = 0;
      }
    }

    shape() {
      const out = M._malloc(8);
      try {
        if (!M._spiraltorch_tensor_shape(this.ptr, out, out + 4)) check(0, "shape");
        return [M.HEAPU32[out >> 2], M.HEAPU32[(out >> 2) + 1]];
      } finally {
        M._free(out);
      }
    }

    elements() {
      return M._spiraltorch_tensor_elements(this.ptr);
    }

    #copy(n, call, what) {
      const buf = M._malloc(Math.max(n, 1) * 4);
      try {
        if (!call(buf, n)) check(0, what);
        return Float32Array.from(M.HEAPF32.subarray(buf >> 2, (buf >> 2) + n));
      } finally {
        M._free(buf);
      }
    }

    data() {
      return this.#copy(this.elements(), (buf, n) => M._spiraltorch_tensor_copy_data(this.ptr, buf, n), "copy_data");
    }

    row(index) {
      return this.#copy(this.shape()[1], (buf, n) => M._spiraltorch_tensor_copy_row(this.ptr, index, buf, n), "copy_row");
    }

    column(index) {
      return this.#copy(this.shape()[0], (buf, n) => M._spiraltorch_tensor_copy_column(this.ptr, index, buf, n), "copy_column");
    }

    add(other) { return new Tensor(check(M._spiraltorch_tensor_add(this.ptr, other.ptr), "add")); }
    sub(other) { return new Tensor(check(M._spiraltorch_tensor_sub(this.ptr, other.ptr), "sub")); }
    hadamard(other) { return new Tensor(check(M._spiraltorch_tensor_hadamard(this.ptr, other.ptr), "hadamard")); }
    matmul(other) { return new Tensor(check(M._spiraltorch_tensor_matmul(this.ptr, other.ptr), "matmul")); }
    scale(s) { return new Tensor(check(M._spiraltorch_tensor_scale(this.ptr, s), "scale")); }
    transpose() { return new Tensor(check(M._spiraltorch_tensor_transpose(this.ptr), "transpose")); }
    reshape(rows, cols) { return new Tensor(check(M._spiraltorch_tensor_reshape(this.ptr, rows, cols), "reshape")); }
    rowSoftmax() { return new Tensor(check(M._spiraltorch_tensor_row_softmax(this.ptr, 0), "row_softmax")); }

    matmulBiasRelu(other, bias) {
      return withFloats(bias, (buf, n) => new Tensor(check(M._spiraltorch_tensor_matmul_bias_relu(this.ptr, other.ptr, buf, n), "matmul_bias_relu")));
    }

    matmulBiasGelu(other, bias) {
      return withFloats(bias, (buf, n) => new Tensor(check(M._spiraltorch_tensor_matmul_bias_gelu(this.ptr, other.ptr, buf, n), "matmul_bias_gelu")));
    }

    matmulBiasAddRelu(other, bias, residual) {
      return withFloats(bias, (buf, n) => new Tensor(check(M._spiraltorch_tensor_matmul_bias_add_relu(this.ptr, other.ptr, buf, n, residual.ptr), "matmul_bias_add_relu")));
    }
  }

  // Partition a gradient's entries by magnitude into above / here / beneath bands.
  // Returns { assignments: Uint8Array, summary: { above, here, beneath, energyAbove, energyHere, energyBeneath } };
  // StRoundtableSummary is three size_t counts (32-bit on wasm32) followed by three f32 energies.
  function roundtableClassify(gradient, aboveK, hereK, beneathK, tolerance) {
    const summaryBytes = 24;
    return withFloats(gradient, (buf, n) => {
      const assign = M._malloc(Math.max(n, 1));
      const summary = M._malloc(summaryBytes);
      try {
        if (!M._spiraltorch_roundtable_classify(buf, n, aboveK, hereK, beneathK, tolerance, assign, summary)) check(0, "roundtable_classify");
        const u = M.HEAPU32.subarray(summary >> 2, (summary >> 2) + 3);
        const f = M.HEAPF32.subarray((summary >> 2) + 3, (summary >> 2) + 6);
        return { assignments: Uint8Array.from(M.HEAPU8.subarray(assign, assign + n)),
                 summary: { above: u[0], here: u[1], beneath: u[2], energyAbove: f[0], energyHere: f[1], energyBeneath: f[2] } };
      } finally {
        M._free(assign);
        M._free(summary);
      }
    });
  }

  return { Tensor, roundtableClassify, lastError, version: () => M.UTF8ToString(M._spiraltorch_version()) };
}

// The C symbols the wrapper calls; build.sh exports exactly these (plus malloc / free).
export const EXPORTED = [
  "spiraltorch_version", "spiraltorch_last_error_length", "spiraltorch_last_error_message", "spiraltorch_clear_last_error",
  "spiraltorch_tensor_from_dense", "spiraltorch_tensor_zeros", "spiraltorch_tensor_random_uniform", "spiraltorch_tensor_random_normal",
  "spiraltorch_tensor_free", "spiraltorch_tensor_shape", "spiraltorch_tensor_elements", "spiraltorch_tensor_copy_data",
  "spiraltorch_tensor_copy_row", "spiraltorch_tensor_copy_column", "spiraltorch_tensor_add", "spiraltorch_tensor_sub",
  "spiraltorch_tensor_hadamard", "spiraltorch_tensor_matmul", "spiraltorch_tensor_scale", "spiraltorch_tensor_transpose",
  "spiraltorch_tensor_reshape", "spiraltorch_tensor_row_softmax", "spiraltorch_tensor_matmul_bias_relu",
  "spiraltorch_tensor_matmul_bias_gelu", "spiraltorch_tensor_matmul_bias_add_relu", "spiraltorch_roundtable_classify",
];
