"""In-tree build of the native sm_100a library.

Every ``csrc/**/*.cu`` file is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` into ``build/obj`` and the
objects are linked into ``spiraltorch_b200/_native/libst_b200.so``.  The library has a
plain C ABI (``extern "C"`` launchers that take raw device pointers and a stream), so it
does not depend on the PyTorch headers and a full rebuild takes well under a minute.

A stamp file next to the ``.so`` holds a hash of the sources; the loader rebuilds only
when the stamp does not match.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parents[2]
CSRC = REPO_ROOT / "csrc"
OBJ_DIR = REPO_ROOT / "build" / "obj"
NATIVE_DIR = REPO_ROOT / "spiraltorch_b200" / "_native"
LIB_PATH = NATIVE_DIR / "libst_b200.so"
STAMP_PATH = NATIVE_DIR / "libst_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-Xptxas", "-v",
]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    p = "/usr/local/cuda/bin/nvcc"
    return p if os.path.exists(p) else None


def sources() -> list[Path]:
    return sorted(CSRC.rglob("*.cu"))


def _all_inputs() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for p in _all_inputs():
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == source_hash()


def _header_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))):
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, hdr_hash: str, verbose: bool) -> tuple[Path, str]:
    rel = src.relative_to(CSRC)
    obj = OBJ_DIR / (str(rel).replace("/", "__") + ".o")
    stamp = obj.with_suffix(".o.stamp")
    key = hashlib.sha256(src.read_bytes() + hdr_hash.encode()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj, ""
    cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {rel}:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(key)
    log = proc.stderr if verbose else ""
    return obj, log


class _BuildLock:
    """Exclusive inter-process lock around check / compile / link / replace.  Under a multi-rank launcher every
    rank loads the library at the same moment; without the lock they would compile into the same object files
    and could link or load a half-written one."""

    def __init__(self, name: str):
        NATIVE_DIR.mkdir(parents=True, exist_ok=True)
        self.path = NATIVE_DIR / name
        self.fh = None

    def __enter__(self):
        import fcntl
        self.fh = open(self.path, "w")
        fcntl.flock(self.fh, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self.fh, fcntl.LOCK_UN)
        self.fh.close()
        return False


def build_native(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile and link the native library if it is missing or stale; return its path."""
    if not force and is_current():
        return LIB_PATH
    with _BuildLock(".build.lock"):
        if not force and is_current():      # another process built it while this one waited
            return LIB_PATH
        return _build_native_locked(force, verbose, jobs)


def _build_native_locked(force: bool, verbose: bool, jobs: int | None) -> Path:
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a native library")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    NATIVE_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for p in OBJ_DIR.glob("*.stamp"):
            p.unlink()
    hdr_hash = _header_hash()
    srcs = sources()
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    logs = []
    with ThreadPoolExecutor(max_workers=max(1, jobs)) as ex:
        results = list(ex.map(lambda s: _compile_one(nvcc, s, hdr_hash, verbose), srcs))
    objs = [str(o) for o, _ in results]
    logs = [l for _, l in results if l]
    tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", str(tmp), *objs, "-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(source_hash())
    if verbose:
        (REPO_ROOT / "build" / "ptxas.log").write_text("\n".join(logs))
        sys.stderr.write("\n".join(logs) + "\n")
    return LIB_PATH


HOST_LIB_PATH = NATIVE_DIR / "libst_host.so"
HOST_STAMP_PATH = NATIVE_DIR / "libst_host.stamp"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-fvisibility=hidden", "-Wall"]


def host_sources() -> list[Path]:
    return sorted((CSRC / "host").glob("*.cpp"))


def _host_hash() -> str:
    h = hashlib.sha256()
    for p in host_sources():
        h.update(p.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()


def build_host(force: bool = False) -> Path:
    """Compile the CUDA-free host runtime (worker pool, rendezvous, loader) with the C++ compiler."""
    if not force and HOST_LIB_PATH.exists() and HOST_STAMP_PATH.exists() and \
            HOST_STAMP_PATH.read_text().strip() == _host_hash():
        return HOST_LIB_PATH
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found: cannot build the host runtime")
    with _BuildLock(".build_host.lock"):
        if not force and HOST_LIB_PATH.exists() and HOST_STAMP_PATH.exists() and \
                HOST_STAMP_PATH.read_text().strip() == _host_hash():
            return HOST_LIB_PATH
        tmp = HOST_LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
        cmd = [cxx, *HOST_FLAGS, *[str(s) for s in host_sources()], "-o", str(tmp)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"host runtime build failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, HOST_LIB_PATH)
        HOST_STAMP_PATH.write_text(_host_hash())
    return HOST_LIB_PATH


if __name__ == "__main__":
    print(build_host(force="--force" in sys.argv))
    path = build_native(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
