"""SpiralK query planner and warp IR."""
import math
import shutil
import subprocess

import pytest

from spiraltorch_b200.kdsl import KdslError
from spiraltorch_b200.kdsl_ir import Filter, QueryPlan, WarpModule, WarpOp, WarpStmt, compile_query


def test_compile_and_execute():
    plan = compile_query("SELECT score WHERE score > 0.5 ORDER BY score DESC LIMIT 3")
    assert plan.selects == ["score"] and plan.filters == [Filter("score", ">", 0.5)] and plan.order == ("score", "desc") and plan.limit == 3
    plan = compile_query("select score,weight where score >= 0.5 and weight != 0.3 order by weight asc;")
    rows = [{"score": 0.7, "weight": 0.1, "x": 1.0}, {"score": 0.2, "weight": 0.5}, {"score": 0.9, "weight": 0.3}, {"score": 0.6, "weight": 0.05}]
    assert plan.execute(rows) == [{"score": 0.6, "weight": 0.05}, {"score": 0.7, "weight": 0.1}]
    assert compile_query("") == QueryPlan() and compile_query("select") .execute(rows) == rows
    assert compile_query("select a order by a").order == ("a", "desc")
    assert compile_query("select a where b <= 2").execute([{"a": 1.0}]) == [{"a": 1.0}]       # a missing column reads as 0
    assert compile_query("select a where b = 0").execute([{"a": 1.0, "b": 1e-17}]) == [{"a": 1.0}]


def test_nan_sorts_last_in_both_directions():
    rows = [{"id": 1.0, "score": math.nan}, {"id": 2.0, "score": math.inf}, {"id": 3.0, "score": -1.0}, {"id": 4.0, "score": -math.inf}]
    assert [r["id"] for r in compile_query("select id order by score asc").execute(rows)] == [4.0, 3.0, 2.0, 1.0]
    assert [r["id"] for r in compile_query("select id order by score desc").execute(rows)] == [2.0, 3.0, 4.0, 1.0]
    assert [r["id"] for r in compile_query("select id order by score desc limit 2").execute(rows)] == [2.0, 3.0]


def test_parse_errors_carry_positions():
    for src, pos in (("score > 1", 0), ("select a where b", 16), ("select a where b ~ 1", 20), ("select a where b > x", 19),
                     ("select a order a", 15), ("select a limit", 14), ("select a limit two", 15)):
        with pytest.raises(KdslError) as e:
            compile_query(src)
        assert str(e.value).endswith(f"at {pos}"), (src, str(e.value))


def test_warp_ir_emits_cuda_intrinsics():
    m = WarpModule()
    m.push(WarpStmt("rotated", "f32", WarpOp("shuffle_xor", "value", "16")))
    m.push(WarpStmt("sum", "f32", WarpOp("reduce_add", "rotated")))
    m.push(WarpStmt("mask", "u32", WarpOp("ballot", "lane < 16")))
    m.push(WarpStmt("all_active", "bool", WarpOp("all", "valid")))
    m.push(WarpStmt("total", "i32", WarpOp("reduce_max", "count")))
    text = m.emit_statements()
    assert "const float rotated = __shfl_xor_sync(0xffffffffu, value, 16);" in text and "const float sum = warp_reduce_add(rotated);" in text
    assert "const unsigned mask = __ballot_sync(0xffffffffu, lane < 16);" in text and "const bool all_active = (__all_sync(0xffffffffu, valid) != 0);" in text
    assert "const int total = __reduce_max_sync(0xffffffffu, count);" in text
    fn = m.emit_function("sg_demo", "float value, int lane, bool valid, int count")
    assert fn.count("warp_reduce_add(T v)") == 1 and "warp_reduce_max" not in m.helpers() and fn.rstrip().endswith("}")
    with pytest.raises(KdslError):
        WarpStmt("x", "f64", WarpOp("all", "p")).emit()
    with pytest.raises(KdslError):
        WarpStmt("x", "f32", WarpOp("shuffle_up", "v")).emit()
    with pytest.raises(KdslError):
        WarpStmt("x", "f32", WarpOp("scan", "v")).emit()


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not on PATH")
def test_emitted_function_compiles_for_sm_100a(tmp_path):
    m = WarpModule()
    m.push(WarpStmt("rotated", "f32", WarpOp("shuffle_xor", "value", "16")))
    m.push(WarpStmt("sum", "f32", WarpOp("reduce_add", "rotated")))
    m.push(WarpStmt("lo", "f32", WarpOp("reduce_min", "rotated")))
    m.push(WarpStmt("votes", "u32", WarpOp("ballot", "valid")))
    m.push(WarpStmt("cnt", "i32", WarpOp("reduce_add", "count")))
    src = tmp_path / "k.cu"
    src.write_text(m.emit_function("sg_demo", "float value, bool valid, int count, float* out", "out[threadIdx.x] = sum + lo + votes + cnt;") +
                   "__global__ void k(float* o) { sg_demo(o[threadIdx.x], true, 1, o); }\n")
    r = subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-c", str(src), "-o", str(tmp_path / "k.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
