"""Documentation stays executable and in sync: README Python blocks run, the capability matrix matches the code."""
import re
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]


def test_readme_python_blocks_run():
    text = (ROOT / "README.md").read_text()
    blocks = re.findall(r"```python\n(.*?)```", text, re.S)
    assert blocks, "README has no python block"
    g = torch.Generator().manual_seed(0)
    import spiraltorch as st
    x = torch.randn(64, 8, generator=g)
    y = torch.sin(x.sum(1, keepdim=True))
    env = {"batches": [(st.Tensor(x[i:i + 16]), st.Tensor(y[i:i + 16])) for i in range(0, 64, 16)]}
    import os
    cwd = os.getcwd()
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        os.chdir(tmp)
        try:
            for block in blocks:
                exec(compile(block, "README.md", "exec"), env)           # noqa: S102 - the README is ours
            assert (Path(tmp) / "weights.json").exists()
        finally:
            os.chdir(cwd)
    assert env["stats"].batches == 4


def test_backend_matrix_doc_in_sync():
    from benchmarks import capability_matrix as cm
    doc = (ROOT / "docs" / "backend_matrix.md").read_text()
    assert cm.render_markdown() in doc, "run `python -m benchmarks.capability_matrix` and refresh docs/backend_matrix.md"
