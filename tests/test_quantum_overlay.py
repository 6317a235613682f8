"""Quantum overlay register (crates/st-qr-studio/src/quantum_overlay.rs)."""
import math

import torch

from spiraltorch_b200 import quantum_overlay as QO
from spiraltorch_b200.theory import MaxwellZPulse


def test_overlay_measures_qubits():
    cfg = QO.QuantumOverlayConfig(-1.0, 4)
    res = QO.ZResonance.from_pulses([MaxwellZPulse(1, 0.5, 0.1, 2.0, (0.2, 0.4, 0.6), 0.7)])
    assert res.spectrum == [0.5] and abs(res.shell_weights[0] - 1.2) < 1e-12 and abs(res.eta_hint - 0.7) < 1e-12
    circ = QO.ZOverlayCircuit.from_config(cfg, res)
    # one shell weight cycled to 24 shells: every shell is 1 / 24
    assert abs(circ.packing_pressure - 1.0 / 24.0) < 1e-12 and abs(circ.eta_bar - math.tanh(0.7 + 1.0 / 24.0)) < 1e-12
    for q in range(4):
        ref = math.tanh(1.0 / 24.0) * 0.65 + abs(math.sin(q / 24.0 * 2 * math.pi) * 0.35) * 0.35
        assert abs(float(circ.weights[q]) - ref) < 1e-12
    m = circ.measure(0.1)
    assert m.active_qubits and m.eta_bar > 0.0 and len(m.policy_logits) == 4
    assert m.policy_logits == sorted(m.policy_logits, reverse=True) and m.active_qubits[0] == 3
    assert circ.measure(99.0).active_qubits == [3] and len(circ.measure(float("nan")).active_qubits) == 4


def test_resonance_and_shell_normalisation():
    assert QO.ZResonance.from_pulses([]).shell_weights == []
    r = QO.ZResonance.from_spectrum([0.5, -1.0, 0.25], -3.0)
    assert r.shell_weights == [0.5, 2.0, 0.75] and r.eta_hint == 0.0
    s = QO.normalize_shells(r, 5)
    assert s.numel() == 5 and abs(float(s.abs().sum()) - 1.0) < 1e-12 and abs(float(s[3] / s[0]) - 1.0) < 1e-12
    assert torch.allclose(QO.normalize_shells(QO.ZResonance(), 3), torch.tensor([1.0, 0.5, 1.0 / 3.0], dtype=torch.float64))
    assert torch.equal(QO.normalize_shells(QO.ZResonance([0.0], 0.0, [0.0]), 2), torch.ones(2, dtype=torch.float64))
    cfg = QO.QuantumOverlayConfig(float("nan"), 0).with_packing_bias(7.0).with_leech_shells(0)
    assert (cfg.curvature, cfg.qubits, cfg.packing_bias, cfg.leech_shells) == (-1.0, 1, 1.0, 1)


def test_batch_matches_single_synthesis():
    cfg = QO.QuantumOverlayConfig(-0.7, 16).with_leech_shells(6)
    rs = [QO.ZResonance.from_spectrum([0.2, 0.9, -0.4], 0.1), QO.ZResonance.from_spectrum([1.0], 0.5), QO.ZResonance(),
          QO.ZResonance.from_spectrum([0.1 * k for k in range(1, 9)], 0.0)]
    batch = QO.ZOverlayCircuit.synthesize_batch(cfg, rs)
    assert batch.shape == (4, 16)
    for row, r in zip(batch, rs):
        assert torch.allclose(row, QO.ZOverlayCircuit.synthesize(cfg, r).weights, atol=1e-12)
