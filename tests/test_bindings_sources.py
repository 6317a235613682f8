"""The Go and Julia wrappers are thin layers over the C ABI: every library symbol they name must exist in the
generated header with the argument count they pass (they cannot be compiled on an image without those toolchains)."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "spiraltorch_b200.h").read_text()
DECLS = {m.group(1): m.group(2) for m in re.finditer(r"\b(spiraltorch_\w+)\(([^)]*)\);", HEADER)}


def _argc(decl: str) -> int:
    decl = decl.strip()
    return 0 if decl in ("", "void") else decl.count(",") + 1


def test_go_binding_names_only_declared_symbols():
    src = (ROOT / "bindings" / "go" / "spiraltorch.go").read_text()
    used = set(re.findall(r"C\.(spiraltorch_\w+)\(", src))
    assert len(used) >= 30 and used <= set(DECLS), sorted(used - set(DECLS))
    for name, args in re.findall(r"C\.(spiraltorch_\w+)\(((?:[^()]|\([^()]*\))*)\)", src):
        depth, count = 0, 1 if args.strip() else 0
        for ch in args:
            depth += ch == "("
            depth -= ch == ")"
            count += ch == "," and depth == 0
        assert count == _argc(DECLS[name]), (name, count, DECLS[name])


def test_julia_binding_names_only_declared_symbols():
    src = (ROOT / "bindings" / "julia" / "src" / "SpiralTorch.jl").read_text()
    used = set(re.findall(r":(spiraltorch_\w+)", src))
    assert len(used) >= 30 and used <= set(DECLS), sorted(used - set(DECLS))
    # ccall argument-type tuples carry one entry per C parameter
    for name, types in re.findall(r"ccall\(_sym\(:(spiraltorch_\w+)\),\s*[\w{}.]+,\s*\(([^)]*)\)", src):
        n = 0 if not types.strip() else len([t for t in types.split(",") if t.strip()])
        assert n == _argc(DECLS[name]), (name, n, DECLS[name])


def test_wasm_binding_names_only_declared_symbols():
    src = (ROOT / "bindings" / "wasm" / "spiraltorch.mjs").read_text()
    used = set(re.findall(r"M\._(spiraltorch_\w+)\(", src))
    exported = set(re.findall(r'"(spiraltorch_\w+)"', src[src.index("export const EXPORTED"):]))
    assert len(used) >= 25 and used <= set(DECLS), sorted(used - set(DECLS))
    assert used == exported, sorted(used ^ exported)                       # the build exports what the wrapper calls, no more
    for name, args in re.findall(r"M\._(spiraltorch_\w+)\(((?:[^()]|\((?:[^()]|\([^()]*\))*\))*)\)", src):
        depth, count = 0, 1 if args.strip() else 0
        for ch in args:
            depth += ch == "("
            depth -= ch == ")"
            count += ch == "," and depth == 0
        assert count == _argc(DECLS[name]), (name, count, DECLS[name])
    # only tensor_abi.cpp is compiled for the browser: nothing the wrapper calls may live in another source file
    for name in used:
        assert re.search(rf"\b{name}\([^)]*\);\s*/\* csrc/host/tensor_abi\.cpp \*/", HEADER), name
