"""The plain-buffer resonance bridge of libst_host (the reference's bindings/cobol_bridge) against the Python text
resonator, and its argument checks."""
import ctypes
from types import SimpleNamespace

import pytest
import torch

from spiraltorch_b200 import text
from spiraltorch_b200.utils import build


@pytest.fixture(scope="module")
def lib():
    handle = ctypes.CDLL(str(build.build_host()))
    handle.st_cobol_new_resonator.restype = ctypes.c_void_p
    handle.st_cobol_new_resonator.argtypes = [ctypes.c_float, ctypes.c_float]
    handle.st_cobol_free_resonator.argtypes = [ctypes.c_void_p]
    handle.st_cobol_describe.restype = ctypes.c_int
    handle.st_cobol_describe.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
    handle.st_cobol_free_string.argtypes = [ctypes.c_void_p]
    return handle


def _describe(lib, h, values):
    arr = (ctypes.c_float * max(len(values), 1))(*values)
    out = ctypes.c_void_p()
    status = lib.st_cobol_describe(h, arr, len(values), ctypes.byref(out))
    if status != 0:
        return status, None
    s = ctypes.string_at(out.value).decode("utf-8")
    lib.st_cobol_free_string(out)
    return status, s


def test_bridge_summary_equals_the_text_resonator(lib):
    h = lib.st_cobol_new_resonator(0.42, 0.58)
    assert h
    for coeffs in ([0.1, -0.3, 0.25, -0.4, 0.55], [0.12, -0.28, 0.44], [3.0]):
        status, summary = _describe(lib, h, coeffs)
        t = torch.tensor([coeffs])
        ref = text.describe_resonance(SimpleNamespace(homotopy_flow=t, functor_linearisation=t, recursive_objective=t, infinity_projection=t,
                                                      infinity_energy=t))
        assert status == 0 and summary == ref and "Above band" in summary and "20.0%" in summary
    status, summary = _describe(lib, h, [0.0, 0.0])
    assert status == 0 and summary.startswith("Resonance geometry is quiescent")
    lib.st_cobol_free_resonator(h)


def test_bridge_rejects_bad_arguments(lib):
    out = ctypes.c_void_p()
    assert lib.st_cobol_describe(None, None, 0, ctypes.byref(out)) == -1
    h = lib.st_cobol_new_resonator(0.2, 0.3)
    assert lib.st_cobol_describe(h, None, 5, ctypes.byref(out)) == -1
    arr = (ctypes.c_float * 1)(1.0)
    assert lib.st_cobol_describe(h, arr, -1, ctypes.byref(out)) == -1 and lib.st_cobol_describe(h, arr, 0, ctypes.byref(out)) == -2
    bad = (ctypes.c_float * 2)(1.0, float("nan"))
    assert lib.st_cobol_describe(h, bad, 2, ctypes.byref(out)) == -2
    lib.st_cobol_free_resonator(h)
    lib.st_cobol_free_resonator(None)
    lib.st_cobol_free_string(None)


def test_resonance_narrative_highlights():
    t = lambda *v: torch.tensor([list(v)])                                             # noqa: E731
    res = SimpleNamespace(homotopy_flow=t(1.0), functor_linearisation=t(2.0), recursive_objective=t(0.0), infinity_projection=t(0.0),
                          infinity_energy=t(1.0))
    n = text.TextResonator().describe_resonance(res)
    assert n.summary.startswith("Here band weaving functor linearisation commanding 66.7%") and "curvature -1.000" in n.summary
    assert n.highlights[:3] == ["Above 16.7%", "Here 66.7%", "Beneath 0.0%"] and "active bands 3" in n.highlights
    quiet = text.resonance_narrative(SimpleNamespace(**{k: t(0.0) for k in ("homotopy_flow", "functor_linearisation", "recursive_objective",
                                                                             "infinity_projection", "infinity_energy")}))
    assert quiet.highlights == ["all bands below activation threshold"]
