"""Maxwell envelopes / sequential Z / Leech projector / RoPE cache (parity:
crates/st-core/src/theory/maxwell.rs, util/math.rs and util/rope_lru.rs unit tests)."""
import math

import pytest
import torch

from spiraltorch_b200.theory import (LeechProjector, MaxwellExpectationError, MaxwellFingerprint, MaxwellSeriesError,
                                     MaxwellZProjector, MeaningGate, RopeLRU, SequentialZ, expected_z_curve,
                                     envelope_series_from_fingerprint, simulate_z_curve)


def test_fingerprint_lambda_and_gate():
    fp = MaxwellFingerprint(0.5, 0.2, 0.8, 20.0, 2.0, math.pi / 3, 4.0)
    assert abs(fp.shielding_factor() - 0.1) < 1e-12 and abs(fp.polarization_alignment() - 0.5) < 1e-12
    assert abs(fp.lambda_() - 0.5 * 0.2 * 0.8 * 0.1 * 2.0 * 0.5 / 4.0) < 1e-15
    assert MaxwellFingerprint(-1, 1, 1, 0, 1, 0, -5).gamma == 0.0
    g = MeaningGate(0.1, 0.4)
    assert g.envelope(5.0) == 0.5 and abs(g.envelope(-0.5) + 0.1) < 1e-12
    s = g.envelope_series([0.0, 1.0, -2.0], [1.0, -1.0, 2.0])
    assert torch.allclose(s, torch.tensor([0.1, -0.5, -0.6], dtype=torch.float64))
    with pytest.raises(MaxwellSeriesError, match="lengths"):
        g.envelope_series([0.0], [1.0, 2.0])
    with pytest.raises(MaxwellSeriesError, match=r"code\[1\]"):
        g.envelope_series([0.0, 0.0], [1.0, math.nan])
    assert torch.allclose(envelope_series_from_fingerprint(fp, 0.0, [0.3], [2.0]), torch.tensor([2 * fp.lambda_()], dtype=torch.float64))


def test_expected_and_simulated_z_curves():
    z = expected_z_curve(4, 2.0, 3.0, 0.5)
    assert torch.allclose(z, 0.75 * torch.sqrt(torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)))
    assert expected_z_curve(0, 1, 1, 1).numel() == 0
    for bad in ((0.0, 1, 1), (1.0, math.inf, 1), (1.0, 1, math.nan)):
        with pytest.raises(MaxwellExpectationError):
            expected_z_curve(3, *bad)
    sim = simulate_z_curve(4000, 1.0, 1.0, 0.2, seed=7)
    assert sim[0] == 0.0 and torch.equal(sim, simulate_z_curve(4000, 1.0, 1.0, 0.2, seed=7))
    assert abs(float(sim[-1]) / float(expected_z_curve(4000, 1.0, 1.0, 0.2)[-1]) - 1.0) < 0.25
    # the closed-form prefix statistics equal the streaming detector
    g = torch.Generator().manual_seed(7)
    x = 0.2 + torch.randn(4000, dtype=torch.float64, generator=g)
    t = SequentialZ()
    assert abs(t.extend(x[:50].tolist()) - float(sim[49])) < 1e-9


def test_sequential_z_and_projector():
    t = SequentialZ()
    assert t.push(1.0) is None and t.variance() is None
    t.push(3.0)
    assert t.mean() == 2.0 and t.variance() == 2.0 and abs(t.z_stat() - 2.0) < 1e-12
    p = MaxwellZProjector(24, 0.5, bias_gain=2.0, min_blocks=3)
    assert p.project(t) is None and p.last_reason == "min_blocks"
    t.push(2.0)
    pulse = p.project(t)
    want = LeechProjector(24, 0.5).enrich(abs(pulse.z_score)) * 2.0
    assert pulse.blocks == 3 and abs(pulse.z_bias - want) < 1e-12 and pulse.band_energy[0] == 2.0 and pulse.band_energy[2] == 0.0
    assert p.last_pulse() is pulse and 0 < pulse.quality() <= 1 and pulse.into_softlogic_feedback(1.0, 2.0)["z_signal"] == pulse.z_bias
    neg = SequentialZ()
    neg.extend([-1.0, -3.0, -2.0])
    assert MaxwellZProjector(24, 0.5).project(neg).z_bias < 0
    assert MaxwellZProjector(24, 0.5, min_z=100.0).project(neg) is None
    flat = SequentialZ()
    flat.extend([1.0, 1.0, 1.0])
    q = MaxwellZProjector(24, 0.5)
    assert q.project(flat) is None and q.last_reason == "undefined_stderr"
    assert LeechProjector(24, 0.0).enrich(3.0) == 0.0
    assert abs(LeechProjector(24, 1.0, 3).ramanujan_ratio - 1.0) < 1e-6


def test_rope_cache_reuses_and_evicts():
    lru = RopeLRU(0)
    assert lru.capacity == 1
    lru = RopeLRU(2)
    c1, s1 = lru.get(0.42, 8)
    c2, s2 = lru.get(0.42 + 1e-12, 8)
    assert c1 is c2 and s1 is s2 and (lru.hits, lru.misses) == (1, 1)
    assert torch.allclose(c1, torch.cos(torch.arange(8) * 0.42), atol=1e-6)
    assert torch.allclose(s1, torch.sin(torch.arange(8) * 0.42), atol=1e-6)
    lru.get(0.5, 8)
    lru.get(0.42, 8)                 # refresh
    lru.get(0.6, 8)                  # evicts 0.5
    assert len(lru) == 2
    assert lru.get(0.42, 8)[0] is c1
    assert lru.get(0.5, 8, dtype=torch.float64)[0].dtype == torch.float64 and lru.misses == 4
