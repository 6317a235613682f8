"""The committed C header lists every exported entry point and compiles as C."""
import re
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_header_is_current_and_complete():
    sys.path.insert(0, str(ROOT / "csrc"))
    import gen_header
    header = (ROOT / "include" / "spiraltorch_b200.h").read_text()
    assert header == gen_header.render(), "run `python csrc/gen_header.py`"
    exported = set()
    for path in (ROOT / "csrc").rglob("*"):
        if path.suffix in (".cu", ".cpp"):
            exported |= set(re.findall(r"^ST_(?:HOST_)?API\s+[^;{(]*?\b(st_\w+)\s*\(", path.read_text(), re.M))
    assert len(exported) > 60
    for name in exported:
        assert re.search(rf"\b{name}\s*\(", header), name
    for must in ("st_gemm_bf16", "st_ag_gemm", "st_gemm_rs", "st_attn_bwd", "st_norm_bwd_noalloc", "st_host_rdv_join",
                 "st_host_pool_submit", "typedef struct StPeerGroup"):
        assert must in header


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "use.c"
    src.write_text('#include "spiraltorch_b200.h"\nint main(void) { struct StPeerGroup g; (void)g; return sizeof(StAttnBwdArgs) > 0 ? 0 : 1; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c", str(src), "-o", str(tmp_path / "use.o")],
                   check=True)
