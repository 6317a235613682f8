"""Tensor-level C ABI of the host library (``spiraltorch_tensor_*`` / ``spiraltorch_runtime_*``), called through
its exported C symbols the way a Go / Julia / C binding would (reference surface:
bindings/spiraltorch-sys/src/lib.rs:130-1640)."""
import ctypes

import pytest
import torch

from spiraltorch_b200.utils import build

c_float_p = ctypes.POINTER(ctypes.c_float)


@pytest.fixture(scope="module")
def lib():
    L = ctypes.CDLL(str(build.build_host()))
    vp = ctypes.c_void_p
    for name in [n for n in ("spiraltorch_tensor_zeros", "spiraltorch_tensor_from_dense", "spiraltorch_tensor_add",
                             "spiraltorch_tensor_sub", "spiraltorch_tensor_hadamard", "spiraltorch_tensor_scale",
                             "spiraltorch_tensor_transpose", "spiraltorch_tensor_reshape", "spiraltorch_tensor_matmul",
                             "spiraltorch_tensor_matmul_with_backend", "spiraltorch_tensor_matmul_bias_relu",
                             "spiraltorch_tensor_matmul_bias_gelu", "spiraltorch_tensor_matmul_bias_add_relu",
                             "spiraltorch_tensor_row_softmax", "spiraltorch_tensor_random_uniform",
                             "spiraltorch_tensor_random_normal", "spiraltorch_tensor_to_dlpack",
                             "spiraltorch_tensor_from_dlpack", "spiraltorch_runtime_new",
                             "spiraltorch_runtime_tensor_matmul", "spiraltorch_runtime_tensor_matmul_bias_gelu",
                             "spiraltorch_runtime_tensor_row_softmax", "spiraltorch_runtime_tensor_add")]:
        getattr(L, name).restype = vp
    L.spiraltorch_version.restype = ctypes.c_char_p
    L.spiraltorch_last_error_length.restype = ctypes.c_size_t
    L.spiraltorch_last_error_message.restype = ctypes.c_size_t
    L.spiraltorch_tensor_elements.restype = ctypes.c_size_t
    L.spiraltorch_runtime_worker_count.restype = ctypes.c_size_t
    for name in ("spiraltorch_tensor_shape", "spiraltorch_tensor_copy_data", "spiraltorch_tensor_copy_row",
                 "spiraltorch_tensor_copy_column", "spiraltorch_roundtable_classify"):
        getattr(L, name).restype = ctypes.c_bool
    return L


def _mk(L, t: torch.Tensor):
    t = t.float().contiguous()
    buf = (ctypes.c_float * t.numel())(*t.reshape(-1).tolist())
    h = L.spiraltorch_tensor_from_dense(ctypes.c_size_t(t.shape[0]), ctypes.c_size_t(t.shape[1]), buf, ctypes.c_size_t(t.numel()))
    assert h, _err(L)
    return ctypes.c_void_p(h)


def _get(L, h) -> torch.Tensor:
    r, c = ctypes.c_size_t(), ctypes.c_size_t()
    assert L.spiraltorch_tensor_shape(h, ctypes.byref(r), ctypes.byref(c))
    n = r.value * c.value
    assert L.spiraltorch_tensor_elements(h) == n
    buf = (ctypes.c_float * n)()
    assert L.spiraltorch_tensor_copy_data(h, buf, ctypes.c_size_t(n))
    return torch.tensor(list(buf)).reshape(r.value, c.value)


def _err(L) -> str:
    buf = ctypes.create_string_buffer(512)
    L.spiraltorch_last_error_message(buf, ctypes.c_size_t(512))
    return buf.value.decode()


def _fvec(v):
    return (ctypes.c_float * len(v))(*v)


def test_elementwise_shape_and_errors(lib):
    assert b"spiraltorch" in lib.spiraltorch_version()
    torch.manual_seed(0)
    a, b = torch.randn(3, 4), torch.randn(3, 4)
    ha, hb = _mk(lib, a), _mk(lib, b)
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_add(ha, hb))), a + b)
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_sub(ha, hb))), a - b)
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_hadamard(ha, hb))), a * b)
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_scale(ha, ctypes.c_float(2.5)))), a * 2.5)
    assert torch.equal(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_transpose(ha))), a.t())
    assert torch.equal(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_reshape(ha, ctypes.c_size_t(2), ctypes.c_size_t(6)))), a.reshape(2, 6))
    row, col = (ctypes.c_float * 4)(), (ctypes.c_float * 3)()
    assert lib.spiraltorch_tensor_copy_row(ha, ctypes.c_size_t(1), row, ctypes.c_size_t(4)) and list(row) == pytest.approx(a[1].tolist())
    assert lib.spiraltorch_tensor_copy_column(ha, ctypes.c_size_t(2), col, ctypes.c_size_t(3)) and list(col) == pytest.approx(a[:, 2].tolist())
    # failures return null / false and leave a message; the next success clears it
    assert not lib.spiraltorch_tensor_reshape(ha, ctypes.c_size_t(5), ctypes.c_size_t(5)) and "cannot reshape" in _err(lib)
    assert not lib.spiraltorch_tensor_add(ha, _mk(lib, torch.zeros(2, 2))) and "shape mismatch" in _err(lib)
    assert not lib.spiraltorch_tensor_add(None, hb) and "null tensor handle" in _err(lib)
    assert not lib.spiraltorch_tensor_zeros(ctypes.c_size_t(0), ctypes.c_size_t(3))
    assert not lib.spiraltorch_tensor_copy_row(ha, ctypes.c_size_t(9), row, ctypes.c_size_t(4))
    assert lib.spiraltorch_tensor_zeros(ctypes.c_size_t(2), ctypes.c_size_t(2)) and lib.spiraltorch_last_error_length() == 0
    for h in (ha, hb):
        lib.spiraltorch_tensor_free(h)


def test_matmul_family_and_runtime(lib):
    torch.manual_seed(1)
    a, b, res = torch.randn(5, 7), torch.randn(7, 6), torch.randn(5, 6)
    bias = torch.randn(6)
    ha, hb, hr = _mk(lib, a), _mk(lib, b), _mk(lib, res)
    ref = a @ b
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_matmul(ha, hb))), ref, atol=1e-5)
    for backend in (0, 1, 2, 3):
        h = lib.spiraltorch_tensor_matmul_with_backend(ha, hb, ctypes.c_int(backend))
        assert torch.allclose(_get(lib, ctypes.c_void_p(h)), ref, atol=1e-5)
    assert not lib.spiraltorch_tensor_matmul_with_backend(ha, hb, ctypes.c_int(4)) and "GPU matmul backends" in _err(lib)
    bv = _fvec(bias.tolist())
    got = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_matmul_bias_relu(ha, hb, bv, ctypes.c_size_t(6))))
    assert torch.allclose(got, torch.relu(ref + bias), atol=1e-5)
    got = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_matmul_bias_gelu(ha, hb, bv, ctypes.c_size_t(6))))
    assert torch.allclose(got, torch.nn.functional.gelu(ref + bias, approximate="tanh"), atol=1e-5)
    got = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_matmul_bias_add_relu(ha, hb, bv, ctypes.c_size_t(6), hr)))
    assert torch.allclose(got, torch.relu(ref + bias + res), atol=1e-5)
    assert not lib.spiraltorch_tensor_matmul_bias_relu(ha, hb, bv, ctypes.c_size_t(5)) and "bias length" in _err(lib)
    assert not lib.spiraltorch_tensor_matmul(hb, hb) and "inner dimensions differ" in _err(lib)
    sm = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_row_softmax(ha, ctypes.c_int(0))))
    assert torch.allclose(sm, torch.softmax(a, -1), atol=1e-6)
    rt = ctypes.c_void_p(lib.spiraltorch_runtime_new(ctypes.c_size_t(3), b"test-pool"))
    assert lib.spiraltorch_runtime_worker_count(rt) == 3
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_runtime_tensor_matmul(rt, ha, hb))), ref, atol=1e-5)
    got = _get(lib, ctypes.c_void_p(lib.spiraltorch_runtime_tensor_matmul_bias_gelu(rt, ha, hb, bv, ctypes.c_size_t(6))))
    assert torch.allclose(got, torch.nn.functional.gelu(ref + bias, approximate="tanh"), atol=1e-5)
    assert torch.allclose(_get(lib, ctypes.c_void_p(lib.spiraltorch_runtime_tensor_row_softmax(rt, ha, ctypes.c_int(0)))),
                          torch.softmax(a, -1), atol=1e-6)
    assert not lib.spiraltorch_runtime_tensor_add(None, ha, ha) and "null runtime handle" in _err(lib)
    lib.spiraltorch_runtime_free(rt)


def test_random_dlpack_and_roundtable(lib):
    u1 = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_random_uniform(ctypes.c_size_t(4), ctypes.c_size_t(50), ctypes.c_float(-1.0),
                                                                       ctypes.c_float(2.0), ctypes.c_uint64(7), ctypes.c_bool(True))))
    u2 = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_random_uniform(ctypes.c_size_t(4), ctypes.c_size_t(50), ctypes.c_float(-1.0),
                                                                       ctypes.c_float(2.0), ctypes.c_uint64(7), ctypes.c_bool(True))))
    assert torch.equal(u1, u2) and u1.min() >= -1.0 and u1.max() < 2.0
    n = _get(lib, ctypes.c_void_p(lib.spiraltorch_tensor_random_normal(ctypes.c_size_t(40), ctypes.c_size_t(50), ctypes.c_float(3.0),
                                                                     ctypes.c_float(0.5), ctypes.c_uint64(1), ctypes.c_bool(True))))
    assert abs(n.mean().item() - 3.0) < 0.05 and abs(n.std().item() - 0.5) < 0.05
    assert not lib.spiraltorch_tensor_random_uniform(ctypes.c_size_t(2), ctypes.c_size_t(2), ctypes.c_float(1.0), ctypes.c_float(1.0),
                                                     ctypes.c_uint64(0), ctypes.c_bool(False))
    a = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    ha = _mk(lib, a)
    cap = ctypes.c_void_p(lib.spiraltorch_tensor_to_dlpack(ha))
    back = ctypes.c_void_p(lib.spiraltorch_tensor_from_dlpack(cap))        # consumes the capsule
    assert torch.equal(_get(lib, back), a)
    grad = [0.9, -0.05, 0.3, -2.0, 0.0, 0.4]
    assign = (ctypes.c_uint8 * 6)()

    class Summary(ctypes.Structure):
        _fields_ = [("above", ctypes.c_size_t), ("here", ctypes.c_size_t), ("beneath", ctypes.c_size_t),
                    ("energy_above", ctypes.c_float), ("energy_here", ctypes.c_float), ("energy_beneath", ctypes.c_float)]
    s = Summary()
    ok = lib.spiraltorch_roundtable_classify(_fvec(grad), ctypes.c_size_t(6), ctypes.c_size_t(2), ctypes.c_size_t(2),
                                             ctypes.c_size_t(2), ctypes.c_float(0.01), assign, ctypes.byref(s))
    assert ok and list(assign) == [0, 2, 1, 0, 1, 1]       # |-2.0| and 0.9 above; 0.0 would be beneath but is within tolerance
    assert (s.above, s.here, s.beneath) == (2, 3, 1) and abs(s.energy_above - 2.9) < 1e-6 and abs(s.energy_beneath - 0.05) < 1e-6
    assert not lib.spiraltorch_roundtable_classify(None, ctypes.c_size_t(6), ctypes.c_size_t(1), ctypes.c_size_t(1),
                                                   ctypes.c_size_t(1), ctypes.c_float(0.0), assign, ctypes.byref(s))
