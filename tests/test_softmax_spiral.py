"""Spiral-consensus softmax and Z-space projection: CPU statement against the closed formulas of the reference
(stub ``_spiral_softmax_hardmax_consensus_python``, softmax_spiral_consensus.wgsl, softmax_zspace_projection.wgsl),
and the fused CUDA kernel against the CPU statement."""
import math

import pytest
import torch

import spiraltorch as st
from spiraltorch_b200.ops import elementwise as E


def test_constants():
    assert abs(E.GOLDEN_RATIO - 1.6180339887) < 1e-9
    assert abs(E.GOLDEN_RATIO_CONJUGATE + E.GOLDEN_RATIO_BIAS - 1.0) < 1e-12
    assert abs(E.RAMANUJAN_PI - math.pi) < 1e-12 and abs(E.RAMANUJAN_RATIO - 1.0) < 1e-12
    assert abs(E.LEECH_SCALE - 0.75 * 0.0019295743094039225 * math.sqrt(24.0)) < 1e-9


def test_consensus_formula_row_by_row():
    torch.manual_seed(0)
    x = torch.randn(4, 7)
    soft, hard, spiral, report = st.Tensor(x).row_softmax_hardmax_spiral()
    p = torch.softmax(x, -1)
    assert torch.allclose(soft.torch(), p, atol=1e-6)
    assert torch.equal(hard.torch().argmax(-1), x.argmax(-1)) and hard.torch().sum().item() == 4
    ent_total = 0.0
    for r in range(4):
        entropy = -sum(v * math.log(v) for v in p[r].tolist() if v > 0)
        enrichment = E.LEECH_SCALE * (entropy * E.RAMANUJAN_RATIO + 1.0 * E.GOLDEN_RATIO)
        want = (1 + enrichment) * (E.GOLDEN_RATIO_CONJUGATE * p[r] + E.GOLDEN_RATIO_BIAS * hard.torch()[r])
        assert torch.allclose(spiral.torch()[r], want, atol=1e-6)
        ent_total += entropy
    assert abs(report["mean_entropy"] - ent_total / 4) < 1e-5
    assert report["mean_hardmass"] == 1.0 and 0.0 < report["spiral_coherence"] < 1.0
    assert set(report) >= {"phi", "phi_conjugate", "phi_bias", "ramanujan_ratio", "ramanujan_delta", "average_enrichment"}


def test_zspace_projection_bands():
    x = torch.zeros(2, 10)
    z = st.Tensor(x).row_softmax_zspace_projection().torch()
    # uniform row of 10: above = floor(10/phi) = 6 columns, here = floor(10/phi^2) = 3 columns
    assert torch.allclose(z[:, 0], torch.full((2,), 0.1), atol=1e-6)
    assert torch.allclose(z[:, 1], torch.full((2,), 0.6), atol=1e-6)
    assert torch.allclose(z[:, 2], torch.full((2,), 0.3), atol=1e-6)
    swirl = sum(0.1 * math.sin(c * E.GOLDEN_ANGLE) for c in range(10))
    assert abs(z[0, 3].item() - swirl) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(3, 5), (17, 300), (4, 5000)])
def test_kernel_matches_cpu_statement(shape):
    torch.manual_seed(1)
    x = torch.randn(*shape) * 3
    cpu = E.row_softmax_spiral(x)
    before = E.launch_count
    gpu = E.row_softmax_spiral(x.cuda())
    assert E.launch_count == before + 1
    for a, b, tol in zip(gpu, cpu, (1e-5, 0, 1e-5, 2e-4, 2e-4)):
        assert (a.cpu() - b).abs().max().item() <= tol + 1e-5 * b.abs().max().item()


def test_nd_indexer_cpu_semantics():
    from spiraltorch_b200.ops import elementwise as E
    pos = torch.arange(24)
    addr, seg = E.nd_indexer(pos, [2, 3, 4], [100, 10, 1], 4, 50)
    want = torch.tensor([100 * (p // 12) + 10 * ((p // 4) % 3) + (p % 4) for p in range(24)])
    assert torch.equal(addr, want) and torch.equal(seg, (want // 50) % 4)
    assert E.nd_indexer(pos[:6], [0, 3, 2], [7, 2, 1], 1, 1)[0].tolist() == [0, 1, 2, 3, 4, 5]          # a zero dimension is skipped
    assert E.nd_indexer(pos.reshape(4, 6), [24], [3], 2, 9)[0].shape == (4, 6)
    for bad in (lambda: E.nd_indexer(pos, [1] * 5, [1] * 5, 1, 1), lambda: E.nd_indexer(pos, [2, 3], [1], 1, 1),
                lambda: E.nd_indexer(pos, [24], [1], 0, 1), lambda: E.nd_indexer(-pos - 1, [24], [1], 1, 1)):
        with pytest.raises(ValueError):
            bad()


@pytest.mark.gpu
def test_nd_indexer_kernel_matches_cpu():
    from spiraltorch_b200.ops import elementwise as E
    torch.manual_seed(0)
    pos = torch.randint(0, 5 * 7 * 11 * 13, (10000,))
    args = ([5, 7, 11, 13], [2002, 143, 13, 1], 8, 640)
    before = E.launch_count
    a_g, s_g = E.nd_indexer(pos.cuda(), *args)
    assert E.launch_count == before + 1
    a_c, s_c = E.nd_indexer(pos, *args)
    assert torch.equal(a_g.cpu(), a_c) and torch.equal(s_g.cpu(), s_c)
