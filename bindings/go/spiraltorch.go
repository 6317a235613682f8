// Package spiraltorch wraps the tensor-level C ABI of libst_host (include/spiraltorch_b200.h): host tensors, a worker
// runtime, the basic algebra with fused epilogues, and the roundtable band classifier.  The API follows the Go binding
// of the reference (bindings/go/spiraltorch.go: Tensor, Runtime, NewTensorFromDense, RoundtableClassify, ...), so code
// written against it builds unchanged.
//
// Build: CGO_CFLAGS="-I<repo>/include" CGO_LDFLAGS="-L<repo>/spiraltorch_b200/_native -lst_host" go build ./...
package spiraltorch

/*
#cgo LDFLAGS: -lst_host
#include <stdlib.h>
#include "spiraltorch_b200.h"
*/
import "C"

import (
	"errors"
	"fmt"
	"runtime"
	"sync"
	"unsafe"
)

// Version reports the library's version string.
func Version() string { return C.GoString(C.spiraltorch_version()) }

func lastError(context string) error {
	n := C.spiraltorch_last_error_length()
	if n == 0 {
		return fmt.Errorf("%s failed", context)
	}
	buf := make([]byte, int(n)+1)
	C.spiraltorch_last_error_message((*C.char)(unsafe.Pointer(&buf[0])), C.size_t(len(buf)))
	C.spiraltorch_clear_last_error()
	return fmt.Errorf("%s: %s", context, string(buf[:n]))
}

// Tensor is a dense row-major float32 matrix owned by the native library.
type Tensor struct {
	ptr *C.SpiralTensor
}

func wrapTensor(ptr *C.SpiralTensor, context string) (*Tensor, error) {
	if ptr == nil {
		return nil, lastError(context)
	}
	t := &Tensor{ptr: ptr}
	runtime.SetFinalizer(t, func(t *Tensor) { t.Close() })
	return t, nil
}

func handle(t *Tensor, context string) (*C.SpiralTensor, error) {
	if t == nil || t.ptr == nil {
		return nil, fmt.Errorf("%s: tensor is closed or nil", context)
	}
	return t.ptr, nil
}

// Close releases the native tensor; further use returns an error.
func (t *Tensor) Close() {
	if t != nil && t.ptr != nil {
		C.spiraltorch_tensor_free(t.ptr)
		t.ptr = nil
	}
}

func seedArgs(seed []uint64) (C.uint64_t, C.bool) {
	if len(seed) > 0 {
		return C.uint64_t(seed[0]), C.bool(true)
	}
	return 0, C.bool(false)
}

func NewZerosTensor(rows, cols int) (*Tensor, error) {
	return wrapTensor(C.spiraltorch_tensor_zeros(C.size_t(rows), C.size_t(cols)), "tensor_zeros")
}

func NewTensorFromDense(rows, cols int, data []float32) (*Tensor, error) {
	if rows < 0 || cols < 0 || len(data) != rows*cols {
		return nil, errors.New("tensor_from_dense: data length does not match rows * cols")
	}
	var p *C.float
	if len(data) > 0 {
		p = (*C.float)(unsafe.Pointer(&data[0]))
	}
	return wrapTensor(C.spiraltorch_tensor_from_dense(C.size_t(rows), C.size_t(cols), p, C.size_t(len(data))), "tensor_from_dense")
}

func NewRandomUniformTensor(rows, cols int, min, max float32, seed ...uint64) (*Tensor, error) {
	s, has := seedArgs(seed)
	return wrapTensor(C.spiraltorch_tensor_random_uniform(C.size_t(rows), C.size_t(cols), C.float(min), C.float(max), s, has), "tensor_random_uniform")
}

func NewRandomNormalTensor(rows, cols int, mean, std float32, seed ...uint64) (*Tensor, error) {
	s, has := seedArgs(seed)
	return wrapTensor(C.spiraltorch_tensor_random_normal(C.size_t(rows), C.size_t(cols), C.float(mean), C.float(std), s, has), "tensor_random_normal")
}

func (t *Tensor) Shape() (int, int, error) {
	h, err := handle(t, "tensor_shape")
	if err != nil {
		return 0, 0, err
	}
	var r, c C.size_t
	if !bool(C.spiraltorch_tensor_shape(h, &r, &c)) {
		return 0, 0, lastError("tensor_shape")
	}
	return int(r), int(c), nil
}

func (t *Tensor) Elements() (int, error) {
	h, err := handle(t, "tensor_elements")
	if err != nil {
		return 0, err
	}
	return int(C.spiraltorch_tensor_elements(h)), nil
}

// CopyDataInto copies the row-major contents into dest and returns the element count.
func (t *Tensor) CopyDataInto(dest []float32) (int, error) {
	n, err := t.Elements()
	if err != nil {
		return 0, err
	}
	if len(dest) < n {
		return 0, fmt.Errorf("tensor_copy_data: destination holds %d values, %d needed", len(dest), n)
	}
	if n > 0 && !bool(C.spiraltorch_tensor_copy_data(t.ptr, (*C.float)(unsafe.Pointer(&dest[0])), C.size_t(n))) {
		return 0, lastError("tensor_copy_data")
	}
	return n, nil
}

func (t *Tensor) Data() ([]float32, error) {
	n, err := t.Elements()
	if err != nil {
		return nil, err
	}
	out := make([]float32, n)
	_, err = t.CopyDataInto(out)
	return out, err
}

func (t *Tensor) CopyRowInto(index int, dest []float32) error {
	h, err := handle(t, "tensor_copy_row")
	if err != nil {
		return err
	}
	if len(dest) == 0 || !bool(C.spiraltorch_tensor_copy_row(h, C.size_t(index), (*C.float)(unsafe.Pointer(&dest[0])), C.size_t(len(dest)))) {
		return lastError("tensor_copy_row")
	}
	return nil
}

func (t *Tensor) CopyColumnInto(index int, dest []float32) error {
	h, err := handle(t, "tensor_copy_column")
	if err != nil {
		return err
	}
	if len(dest) == 0 || !bool(C.spiraltorch_tensor_copy_column(h, C.size_t(index), (*C.float)(unsafe.Pointer(&dest[0])), C.size_t(len(dest)))) {
		return lastError("tensor_copy_column")
	}
	return nil
}

func binary(a, b *Tensor, context string, op func(x, y *C.SpiralTensor) *C.SpiralTensor) (*Tensor, error) {
	x, err := handle(a, context)
	if err != nil {
		return nil, err
	}
	y, err := handle(b, context)
	if err != nil {
		return nil, err
	}
	out, err := wrapTensor(op(x, y), context)
	runtime.KeepAlive(a)
	runtime.KeepAlive(b)
	return out, err
}

func (t *Tensor) Add(o *Tensor) (*Tensor, error) {
	return binary(t, o, "tensor_add", func(x, y *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_add(x, y) })
}

func (t *Tensor) Sub(o *Tensor) (*Tensor, error) {
	return binary(t, o, "tensor_sub", func(x, y *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_sub(x, y) })
}

func (t *Tensor) Hadamard(o *Tensor) (*Tensor, error) {
	return binary(t, o, "tensor_hadamard", func(x, y *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_hadamard(x, y) })
}

func (t *Tensor) Matmul(o *Tensor) (*Tensor, error) {
	return binary(t, o, "tensor_matmul", func(x, y *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_matmul(x, y) })
}

// MatmulBiasRelu computes relu(t·o + bias) in one call; bias has one value per output column.
func (t *Tensor) MatmulBiasRelu(o *Tensor, bias []float32) (*Tensor, error) {
	if len(bias) == 0 {
		return nil, errors.New("tensor_matmul_bias_relu: empty bias")
	}
	return binary(t, o, "tensor_matmul_bias_relu", func(x, y *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_tensor_matmul_bias_relu(x, y, (*C.float)(unsafe.Pointer(&bias[0])), C.size_t(len(bias)))
	})
}

// MatmulBiasGelu computes gelu(t·o + bias) in one call.
func (t *Tensor) MatmulBiasGelu(o *Tensor, bias []float32) (*Tensor, error) {
	if len(bias) == 0 {
		return nil, errors.New("tensor_matmul_bias_gelu: empty bias")
	}
	return binary(t, o, "tensor_matmul_bias_gelu", func(x, y *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_tensor_matmul_bias_gelu(x, y, (*C.float)(unsafe.Pointer(&bias[0])), C.size_t(len(bias)))
	})
}

func unary(t *Tensor, context string, op func(x *C.SpiralTensor) *C.SpiralTensor) (*Tensor, error) {
	x, err := handle(t, context)
	if err != nil {
		return nil, err
	}
	out, err := wrapTensor(op(x), context)
	runtime.KeepAlive(t)
	return out, err
}

func (t *Tensor) Scale(v float32) (*Tensor, error) {
	return unary(t, "tensor_scale", func(x *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_scale(x, C.float(v)) })
}

func (t *Tensor) Transpose() (*Tensor, error) {
	return unary(t, "tensor_transpose", func(x *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_transpose(x) })
}

func (t *Tensor) Reshape(rows, cols int) (*Tensor, error) {
	return unary(t, "tensor_reshape", func(x *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_tensor_reshape(x, C.size_t(rows), C.size_t(cols))
	})
}

func (t *Tensor) RowSoftmax() (*Tensor, error) {
	return unary(t, "tensor_row_softmax", func(x *C.SpiralTensor) *C.SpiralTensor { return C.spiraltorch_tensor_row_softmax(x, 0) })
}

// Runtime is a pool of worker threads on which tensor operations run.
type Runtime struct {
	ptr *C.RuntimeHandle
}

func NewRuntime(workerThreads int, threadName string) (*Runtime, error) {
	var name *C.char
	if threadName != "" {
		name = C.CString(threadName)
		defer C.free(unsafe.Pointer(name))
	}
	ptr := C.spiraltorch_runtime_new(C.size_t(workerThreads), name)
	if ptr == nil {
		return nil, lastError("runtime_new")
	}
	r := &Runtime{ptr: ptr}
	runtime.SetFinalizer(r, func(r *Runtime) { r.Close() })
	return r, nil
}

func (r *Runtime) Close() {
	if r != nil && r.ptr != nil {
		C.spiraltorch_runtime_free(r.ptr)
		r.ptr = nil
	}
}

func (r *Runtime) WorkerCount() (int, error) {
	if r == nil || r.ptr == nil {
		return 0, errors.New("runtime_worker_count: runtime is closed")
	}
	return int(C.spiraltorch_runtime_worker_count(r.ptr)), nil
}

func (r *Runtime) binary(a, b *Tensor, context string, op func(rt *C.RuntimeHandle, x, y *C.SpiralTensor) *C.SpiralTensor) (*Tensor, error) {
	if r == nil || r.ptr == nil {
		return nil, fmt.Errorf("%s: runtime is closed", context)
	}
	return binary(a, b, context, func(x, y *C.SpiralTensor) *C.SpiralTensor { return op(r.ptr, x, y) })
}

func (r *Runtime) Add(a, b *Tensor) (*Tensor, error) {
	return r.binary(a, b, "runtime_tensor_add", func(rt *C.RuntimeHandle, x, y *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_runtime_tensor_add(rt, x, y)
	})
}

func (r *Runtime) Sub(a, b *Tensor) (*Tensor, error) {
	return r.binary(a, b, "runtime_tensor_sub", func(rt *C.RuntimeHandle, x, y *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_runtime_tensor_sub(rt, x, y)
	})
}

func (r *Runtime) Hadamard(a, b *Tensor) (*Tensor, error) {
	return r.binary(a, b, "runtime_tensor_hadamard", func(rt *C.RuntimeHandle, x, y *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_runtime_tensor_hadamard(rt, x, y)
	})
}

func (r *Runtime) Matmul(a, b *Tensor) (*Tensor, error) {
	return r.binary(a, b, "runtime_tensor_matmul", func(rt *C.RuntimeHandle, x, y *C.SpiralTensor) *C.SpiralTensor {
		return C.spiraltorch_runtime_tensor_matmul(rt, x, y)
	})
}

// TensorPair is one (left, right) operand pair of a parallel batch.
type TensorPair struct {
	Lhs, Rhs *Tensor
}

func (r *Runtime) parallel(pairs []TensorPair, concurrency int, op func(a, b *Tensor) (*Tensor, error)) ([]*Tensor, error) {
	if concurrency <= 0 {
		concurrency = runtime.NumCPU()
	}
	out := make([]*Tensor, len(pairs))
	errs := make([]error, len(pairs))
	sem := make(chan struct{}, concurrency)
	var wg sync.WaitGroup
	for i, p := range pairs {
		wg.Add(1)
		sem <- struct{}{}
		go func(i int, p TensorPair) {
			defer wg.Done()
			defer func() { <-sem }()
			out[i], errs[i] = op(p.Lhs, p.Rhs)
		}(i, p)
	}
	wg.Wait()
	for _, err := range errs {
		if err != nil {
			for _, t := range out {
				t.Close()
			}
			return nil, err
		}
	}
	return out, nil
}

func (r *Runtime) ParallelMatmul(pairs []TensorPair, concurrency int) ([]*Tensor, error) {
	return r.parallel(pairs, concurrency, r.Matmul)
}

func (r *Runtime) ParallelAdd(pairs []TensorPair, concurrency int) ([]*Tensor, error) {
	return r.parallel(pairs, concurrency, r.Add)
}

func (r *Runtime) ParallelHadamard(pairs []TensorPair, concurrency int) ([]*Tensor, error) {
	return r.parallel(pairs, concurrency, r.Hadamard)
}

// RoundtableBand is the band a gradient entry was assigned to.
type RoundtableBand uint8

const (
	BandAbove RoundtableBand = iota
	BandHere
	BandBeneath
)

func (b RoundtableBand) String() string {
	switch b {
	case BandAbove:
		return "above"
	case BandHere:
		return "here"
	case BandBeneath:
		return "beneath"
	}
	return "unknown"
}

// RoundtableSummary counts the entries and the energy of each band.
type RoundtableSummary struct {
	Above, Here, Beneath                     int
	EnergyAbove, EnergyHere, EnergyBeneath float32
}

// RoundtableClassify splits a gradient into the above / here / beneath bands (top-k, within tolerance, bottom-k).
func RoundtableClassify(gradient []float32, aboveK, hereK, beneathK int, tolerance float32) ([]RoundtableBand, RoundtableSummary, error) {
	if len(gradient) == 0 {
		return nil, RoundtableSummary{}, nil
	}
	assign := make([]RoundtableBand, len(gradient))
	var s C.StRoundtableSummary
	ok := C.spiraltorch_roundtable_classify((*C.float)(unsafe.Pointer(&gradient[0])), C.size_t(len(gradient)), C.size_t(aboveK), C.size_t(hereK),
		C.size_t(beneathK), C.float(tolerance), (*C.uint8_t)(unsafe.Pointer(&assign[0])), &s)
	if !bool(ok) {
		return nil, RoundtableSummary{}, lastError("roundtable_classify")
	}
	return assign, RoundtableSummary{int(s.above), int(s.here), int(s.beneath), float32(s.energy_above), float32(s.energy_here), float32(s.energy_beneath)}, nil
}
