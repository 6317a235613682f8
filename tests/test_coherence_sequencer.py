"""Z-space coherence sequencer: measurement engine, aggregate against the explicit recurrences, pre-discard policy and
regulator, diagnostics / classification contract, language bridges and the stage-trace recorder.  Scenarios follow the
behaviours exercised by crates/st-nn/src/zspace_coherence/{coherence_engine,sequencer,trace}.rs and
crates/st-core/src/inference/zspace_coherence.rs."""
import json
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200 import zspace_coherence as zc
from spiraltorch_b200.language import ConceptHint, MaxwellDesireBridge, NarrativeHint, SemanticBridge
from spiraltorch_b200.nn import coherence as C
from spiraltorch_b200.theory import MaxwellZPulse
from spiraltorch_b200.topos import OpenCartesianTopos


def _seq(dim=128, heads=8, curvature=-1.0):
    return C.ZSpaceCoherenceSequencer(dim, heads, curvature, OpenCartesianTopos(curvature, 1e-5, 10.0, 256, 8192))


def _t(data, rows=1):
    return st.Tensor._wrap(torch.tensor(data, dtype=torch.float32).reshape(rows, -1))


# ---- contract --------------------------------------------------------------------------------------------------------
def test_projection_contract_matches_formulas():
    h = 1.0296530140645737
    d = zc.DiagnosticsInput(0.25, h, 0.7, -0.12, 0.4, [0.5, 0.3, 0.2, 0.0], 3, 1, 0)
    p = zc.project(d, [0.5, 0.3, 0.2, 0.0])
    conc, hn = (0.38 - 0.25) / 0.75, h / math.log(4.0)
    assert p.contract_version == "spiraltorch.zspace_coherence_projection.v2"
    assert p.derived.distribution_source == "normalized_weights"
    assert p.classification.label == "cascade_imbalance"
    assert p.classification.reason == "dominant_energy_ratio_at_or_above_cascade_min"
    assert p.control.spectral_radius == pytest.approx(conc, abs=1e-14)
    assert p.control.spectral_entropy == pytest.approx(hn, abs=1e-14)
    assert p.control.spectral_pressure == pytest.approx(0.7 * (1 - hn), abs=1e-14)
    assert p.partial["speed"] == pytest.approx(math.tanh(conc), abs=1e-14)
    assert p.partial["stability"] == pytest.approx(math.tanh(1 - 2 * hn), abs=1e-14)
    assert p.partial["memory"] == pytest.approx(math.tanh(-0.12), abs=1e-14)
    assert p.partial["coherence_entropy_residual"] == pytest.approx(0.0, abs=1e-14)
    assert p.partial["coherence_channels"] == 4.0
    for k in p.partial:
        if k.startswith("coherence_"):
            assert zc.canonical_metric_name(k) == k
    d.discarded_channels = None
    q = zc.project(d, [0.5, 0.3, 0.2, 0.0])
    assert q.partial["coherence_preserved"] == 3.0 and q.partial["coherence_discarded"] == 1.0


def test_projection_contract_rejects_inconsistent_evidence():
    good = dict(mean_coherence=0.25, coherence_entropy=1.0296530140645737, energy_ratio=0.7, z_bias=0.0, fractional_order=0.4,
                normalized_weights=[0.5, 0.3, 0.2, 0.0], preserved_channels=3, discarded_channels=1, dominant_channel=0)
    for patch, code in ((dict(coherence_entropy=0.5), "inconsistent_distribution_metric"), (dict(preserved_channels=4, discarded_channels=0), "inconsistent_channel_support"),
                        (dict(dominant_channel=1), "inconsistent_dominant_channel"), (dict(dominant_channel=9), "dominant_out_of_range"),
                        (dict(normalized_weights=[0.5, 0.3, 0.3, 0.0]), "invalid_weight_mass"), (dict(energy_ratio=1.5), "scalar_out_of_range"),
                        (dict(z_bias=float("nan")), "non_finite_scalar")):
        with pytest.raises(zc.CoherenceProjectionError) as e:
            zc.project(zc.DiagnosticsInput(**{**good, **patch}), [0.5, 0.3, 0.2, 0.0])
        assert e.value.code == code
    with pytest.raises(zc.CoherenceProjectionError):
        zc.project(zc.DiagnosticsInput(**good), [0.5, 0.3, 0.2, 0.0], config=zc.ProjectionConfig(speed_gain=-1.0))
    # entropy alone (no weights): no classification, concentration = 1 - normalized entropy
    p = zc.project(zc.DiagnosticsInput(0.25, math.log(4.0) / 2, 0.5, 0.0, 0.3, [], 4, 0, None))
    assert p.classification is None and p.control is None and p.derived.concentration == pytest.approx(0.5)


def test_classification_and_swap_invariance():
    assert zc.is_swap_invariant([0.5, 0.5, 0.5]) and not zc.is_swap_invariant([float("nan")] * 2)
    assert not zc.is_swap_invariant([]) and not zc.is_swap_invariant([0.5, 0.2, 0.5])
    assert zc.classify(0.0, True).label == "background"
    assert zc.classify(0.3, True).label == "symmetric_pulse"
    assert zc.classify(0.7, False).label == "cascade_imbalance"
    assert zc.classify(0.4, False).label == "diffuse_drift"
    assert zc.classify(0.4, False, zc.ClassificationPolicy(0.5, 0.9)).label == "background"
    with pytest.raises(zc.CoherenceProjectionError):
        zc.classify(0.4, False, zc.ClassificationPolicy(0.9, 0.5))
    for n in (2, 16, 1024):                                 # uniform -> entropy 1, concentration 0 whatever the width
        s = zc.summarize_distribution([1.0 / n] * n)
        assert s.normalized_entropy == pytest.approx(1.0) and s.concentration == pytest.approx(0.0, abs=1e-9)
        s = zc.summarize_distribution([1.0] + [0.0] * (n - 1))
        assert s.normalized_entropy == 0.0 and s.concentration == 1.0 and s.effective_channels == 1.0
    w = zc.build_distribution_witness([0.25] * 4)
    assert zc.validate_distribution_observation(w, 4, 2).channels == 4
    w.kind = "other"
    with pytest.raises(zc.CoherenceProjectionError):
        zc.validate_distribution_witness(w)


# ---- engine ----------------------------------------------------------------------------------------------------------
def test_engine_weights_sum_to_one_and_follow_energy():
    eng = C.CoherenceEngine(128, -1.0)
    assert eng.num_channels == 2
    x = torch.zeros(3, 128)
    x[:, 64:] = 2.0
    x[:, :64] = 0.5
    w = eng.measure_phases(x)
    assert sum(w) == pytest.approx(1.0, abs=1e-5) and w[1] == pytest.approx(0.8, abs=1e-5)
    eng.register_linguistic_profile(C.DomainLinguisticProfile("membrane", emphasis=2.0))      # favours low channels
    w2 = eng.measure_phases(x)
    assert w2[0] > w[0]
    eng.clear_linguistic_profiles()
    eng.set_backend("cufft")
    assert eng.is_accelerated() and eng.backend.capabilities()["gpu"]
    assert eng.measure_phases(x) == pytest.approx(w, abs=1e-6)       # a uniform backend bias cancels in the normalisation
    with pytest.raises(st.TensorError):
        eng.measure_phases(torch.zeros(2, 64))
    with pytest.raises(st.TensorError):
        C.CoherenceEngine(64, 0.5)


def test_linguistic_contour_and_channel_reports():
    eng = C.CoherenceEngine(64, -4.0, 4)
    c = eng.derive_linguistic_contour([0.0, 0.0, 0.0, 1.0])
    assert c.coherence_strength == 1.0 and c.prosody_index == 1.0 and c.timbre_spread == 0.0 and c.articulation_bias == 2.0
    u = eng.derive_linguistic_contour([1.0] * 4)
    assert u.coherence_strength == pytest.approx(0.25) and u.prosody_index == pytest.approx(0.5)
    eng.register_linguistic_profile(C.DomainLinguisticProfile("grain_boundary", descriptor="rising"))
    eng.register_linguistic_profile(C.DomainLinguisticProfile("membrane", descriptor="falling"))
    reps = eng.describe_channels([0.25] * 4)
    assert reps[0].dominant_concept == "membrane" and reps[3].dominant_concept == "grain_boundary"
    assert reps[3].descriptor == "rising" and reps[0].backend.label() == "pure_rust"
    prof = C.DomainLinguisticProfile("custom", harmonic_bias=[2.0, 3.0])
    assert prof.harmonic_multiplier(5, 8) == 3.0 and prof.harmonic_bias_len() == 2
    with pytest.raises(st.TensorError):
        C.DomainLinguisticProfile("membrane", emphasis=0.0)
    with pytest.raises(st.TensorError):
        eng.derive_linguistic_contour([0.5, 0.5])


# ---- aggregate -------------------------------------------------------------------------------------------------------
def _explicit_aggregate(x, weights, order, cw):
    out = torch.zeros_like(x)
    norm = max(sum(max(w, 0.0) for w in weights), 1e-6)
    for r in range(x.shape[0]):
        row = [x[r, j].item() * max(weights[j // cw], 0.0) / norm for j in range(x.shape[1])]
        acc = row[0]
        for j in range(1, len(row)):
            acc += order * (row[j] - acc)
            row[j] = acc
        acc = row[-1]
        for j in range(len(row) - 2, -1, -1):
            acc += order * (row[j] - acc)
            row[j] = acc
        out[r] = torch.tensor(row)
    return out


def test_aggregate_matches_explicit_recurrences_and_forward_path():
    torch.manual_seed(0)
    seq = _seq(64, 4, -1.0)
    x = torch.randn(3, 64) * 0.3
    z = seq.project_to_zspace(st.Tensor._wrap(x))
    assert float(z.torch().norm(dim=1).max()) < 1.0                      # inside the unit ball
    w = seq.coherence_engine.measure_phases(z)
    agg = seq.geometric_aggregate(z, w).torch()
    ref = seq.topos.saturate(_explicit_aggregate(z.torch(), w, seq.fractional_order(), 8))
    assert torch.allclose(agg, ref, atol=1e-6)
    out, coh = seq.forward_with_coherence(st.Tensor._wrap(x))
    assert out.shape() == (3, 64) and torch.allclose(out.torch(), agg, atol=1e-7) and coh == w
    assert torch.equal(seq.forward(st.Tensor._wrap(x)).torch(), out.torch())
    # non-finite / negative weights are repaired, not propagated
    bad = list(w)
    bad[0], bad[1] = float("nan"), -1.0
    _, _, _, _, repairs = seq._aggregate(z, bad)
    assert repairs == (1, 1) and bool(torch.isfinite(seq.geometric_aggregate(z, bad).torch()).all())
    assert seq.fractional_order() == pytest.approx(0.5) and seq.canonical_domain_concept() == "membrane"
    assert _seq(192, 24, -1.0).canonical_domain_concept() == "neuronal_pattern"
    with pytest.raises(st.TensorError):
        C.ZSpaceCoherenceSequencer(130, 8, -1.0, OpenCartesianTopos(-1.0, 1e-5, 10.0, 256, 8192))
    with pytest.raises(st.TensorError):
        C.ZSpaceCoherenceSequencer(128, 8, -0.5, OpenCartesianTopos(-1.0, 1e-5, 10.0, 256, 8192))


def test_coherent_aggregation_emphasises_stronger_channels():
    seq = _seq()
    data = [0.05] * 128
    for j in range(96, 128):
        data[j] = 0.8
    out, coh, diag = seq.forward_with_diagnostics(_t(data))
    a = out.torch()[0]
    assert float(a[100:].abs().mean()) > 10 * float(a[:64].abs().mean())
    assert diag.dominant_channel >= 12 and diag.preserved_channels() == 16 and diag.discarded_channels() == 0
    assert len(diag.channel_reports) == seq.maxwell_channels() == 16
    assert diag.z_bias < 0                                               # the mass sits in the last third of the channels
    assert diag.observation().is_signature
    assert diag.control_summary().spectral_entropy == pytest.approx(diag.distribution_summary().normalized_entropy)
    partial = diag.project_to_zspace_partial(contour=seq.emit_linguistic_contour(seq.project_to_zspace(_t(data)))).partial
    assert partial["coherence_channels"] == 16.0 and "coherence_prosody" in partial


def test_diagnostics_observation_labels():
    def diag(weights, normalized, energy_ratio):
        return C.CoherenceDiagnostics(weights, normalized, 1.0, 0.5, 0, 0, 0 if weights else None, sum(weights) / max(len(weights), 1),
                                      0.0, energy_ratio, 0.0, st.Tensor._wrap(torch.zeros(1, 4)))
    assert not diag([], [], 0.0).observation().is_signature and diag([], [], 0.0).observation().lift_to_label() == "background"
    sym = diag([0.2] * 4, [0.25] * 4, 0.3).observation()
    assert sym.lift_to_label() == "symmetric_pulse" and sym.signature.normalized_entropy > 0.99
    assert sym.signature.concentration < 1e-6 and sym.signature.channels == 4 and sym.signature.classification_reason == "swap_invariant"
    assert diag([0.8, 0.05, 0.05, 0.05], [0.8, 0.07, 0.07, 0.06], 0.85).observation().lift_to_label() == "cascade_imbalance"
    zero = diag([0.25] * 4, [0.25] * 4, 0.0)
    assert not zero.observation().is_signature
    assert zero.observation_with_policy(zc.ClassificationPolicy(0.0, 0.7)).lift_to_label() == "background"


# ---- pre-discard -----------------------------------------------------------------------------------------------------
def test_pre_discard_culls_weak_channels_and_journal_records_history():
    seq = _seq()
    seq.enable_pre_discard(C.PreDiscardPolicy(0.35).with_energy_floor(1e-4).with_min_channels(2))
    data = [0.02] * 128
    for j in range(96, 128):
        data[j] = 0.9
    _, coh, diag = seq.forward_with_diagnostics(_t(data))
    tel = diag.pre_discard
    assert diag.discarded_channels() > 0 and diag.preserved_channels() < seq.maxwell_channels()
    assert tel.discarded == diag.discarded_channels() and not tel.used_fallback
    assert sum(coh) == pytest.approx(1.0, abs=1e-5) and tel.survivor_energy_ratio > 0.9
    assert tel.preserved_ratio == pytest.approx(diag.preserved_channels() / 16)
    snaps = seq.pre_discard_snapshots()
    assert len(snaps) == 1 and snaps[0].step == 0 and len(snaps[0].survivors) == tel.preserved
    seq.configure_pre_discard_memory(2)
    for _ in range(3):
        seq.forward(_t(data))
    snaps = seq.pre_discard_snapshots()
    assert [s.step for s in snaps] == [2, 3]
    seq.clear_pre_discard_snapshots()
    assert seq.pre_discard_snapshots() == []
    seq.disable_pre_discard()
    _, _, after = seq.forward_with_diagnostics(_t(data))
    assert after.discarded_channels() == 0 and after.pre_discard is None


def test_pre_discard_policy_edge_cases():
    p = C.PreDiscardPolicy(0.5)
    f, tel, surv, disc = p.apply([float("nan"), -1.0, 0.4, 0.1])
    assert surv == [2] and disc == [0, 1, 3] and f == [0.0, 0.0, 1.0, 0.0]
    assert (tel.repaired_non_finite, tel.repaired_negative) == (1, 1) and tel.repairs_total == 2
    f, tel, surv, _ = p.apply([0.0, 0.0, 0.0])
    assert tel.used_fallback and f == pytest.approx([1 / 3] * 3) and surv == [0, 1, 2]
    f, tel, _, _ = C.PreDiscardPolicy(0.0).with_min_channels(3).apply([0.5, 0.3, 0.1, 0.1])
    assert tel.preserved == 3 and f[3] == 0.0
    assert p.apply([])[1].used_fallback
    assert C.PreDiscardPolicy(7.0).dominance_ratio == 1.0
    with pytest.raises(st.TensorError):
        C.PreDiscardPolicy(-0.1)
    with pytest.raises(st.TensorError):
        C.PreDiscardPolicy(0.5, energy_floor=float("inf"))


def _tel(preserved, discarded, surv_e=0.9, disc_e=0.1, fallback=False, dominant=0.5):
    return C.PreDiscardTelemetry(0.3, 0.0, discarded, preserved, fallback, surv_e, disc_e, dominant)


def test_pre_discard_regulator_control_law():
    reg = C.PreDiscardRegulator(0.25, 0.8)
    reg.observe(_tel(12, 4))                                  # keeps 75 % of channels against a 25 % target
    assert reg.offset < 0 and reg.observations == 1
    assert reg.next_policy(C.PreDiscardPolicy(0.3)).dominance_ratio < 0.3
    pen = C.PreDiscardRegulator(1.0, 1.0).with_fallback_penalty(0.15)
    pen.observe(_tel(8, 0, 1.0, 0.0, fallback=True))
    plain = C.PreDiscardRegulator(1.0, 1.0).with_fallback_penalty(0.0)
    plain.observe(_tel(8, 0, 1.0, 0.0, fallback=True))
    assert pen.offset == pytest.approx(-0.15) and plain.offset == 0.0
    dead = C.PreDiscardRegulator(0.5, 0.9).with_deadband(0.2)
    dead.observe(_tel(9, 7))
    assert dead.offset == 0.0
    mom, flat = C.PreDiscardRegulator(0.3, 0.9).with_momentum(1.0), C.PreDiscardRegulator(0.3, 0.9)
    for r in (mom, flat):
        r.observe(_tel(8, 8))
        r.observe(_tel(14, 2))
    assert mom.offset < flat.offset
    dec = C.PreDiscardRegulator(0.5, 0.9).with_equilibrium_decay(0.5).with_smoothing(1.0)
    dec.observe(_tel(14, 2))
    before = dec.offset
    dec.observe(_tel(8, 8, 0.9, 0.1))
    assert abs(dec.offset) < abs(before)
    lo, hi = C.PreDiscardRegulator(0.3, 0.9).with_confidence_scaling(0.5, 0.0), C.PreDiscardRegulator(0.3, 0.9).with_confidence_scaling(0.0, 2.0)
    base = C.PreDiscardRegulator(0.3, 0.9)
    for r in (lo, hi, base):
        r.observe(_tel(12, 4, dominant=0.25))
    assert abs(lo.offset) < abs(base.offset) < abs(hi.offset)
    integ = C.PreDiscardRegulator(0.3, 0.9).with_integral_control(0.5, 2.0, 0.0).with_max_step(1.0).with_bounds(-5.0, 5.0)
    ref = C.PreDiscardRegulator(0.3, 0.9).with_max_step(1.0).with_bounds(-5.0, 5.0)
    for _ in range(3):
        integ.observe(_tel(12, 4))
        ref.observe(_tel(12, 4))
    assert integ.offset < ref.offset
    for bad in (lambda: C.PreDiscardRegulator(-0.1, 0.5), lambda: base.with_trend_smoothing(1.5), lambda: base.with_max_step(0.0),
                lambda: base.with_bounds(1.0, -1.0), lambda: base.with_error_weights(0.0, 0.0), lambda: base.with_aggressiveness(0.0)):
        with pytest.raises(st.TensorError):
            bad()


def test_adaptive_regulator_changes_the_sequencers_policy_over_time():
    seq = _seq()
    seq.enable_pre_discard(C.PreDiscardPolicy(0.9), C.PreDiscardRegulator(0.25, 0.5).with_aggressiveness(1.0))
    data = [0.02 + 0.005 * (j // 8) for j in range(128)]
    first = seq.forward_with_diagnostics(_t(data))[2].pre_discard
    for _ in range(4):
        last = seq.forward_with_diagnostics(_t(data))[2].pre_discard
    assert seq.pre_discard_regulator().observations == 5
    assert last.dominance_ratio < first.dominance_ratio and last.preserved < first.preserved


# ---- language bridges, trace -----------------------------------------------------------------------------------------
def _pulse():
    return MaxwellZPulse(6, 0.32, 0.07, 3.4, (0.5, 0.3, 0.1), 0.41)


def test_maxwell_desire_bridge_and_narrative_hint():
    bridge = MaxwellDesireBridge().with_smoothing(0.05).with_magnitude_floor(0.2)
    bridge.register_channel("alpha", [(0, 0.6), (2, 0.4)])
    hint = bridge.hint_for("alpha", _pulse())
    assert hint.window == [(0, pytest.approx(0.65 * 3.4)), (2, pytest.approx(0.45 * 3.4))]
    assert bridge.narrative_for("alpha", _pulse()) is None and bridge.hint_for("beta", _pulse()) is None
    bridge.register_channel("beta", [(1, 1.0)], tags=[" glimmer ", "braid", "braid"], gain=0.5)
    assert bridge.narrative_tags("beta") == ["braid", "glimmer"]
    n = bridge.narrative_for("beta", _pulse())
    assert n.intensity == pytest.approx(1.7) and n.dominant_tag() in ("braid", "glimmer")
    assert n.coherence == pytest.approx(0.6 / 0.900001, rel=1e-5) and n.decoherence == pytest.approx(0.07 / 1.07)
    s = n.summary()
    assert s.emphasis == pytest.approx(1.7 * n.coherence * (1 - n.decoherence)) and s.describe().startswith("[beta] tag `")
    assert NarrativeHint("c", [], 0.0).summary().describe().startswith("[c] neutral")
    for bad in (("", [(0, 1.0)]), ("x", []), ("x", [(0, -1.0)]), ("x", [(0, float("nan"))])):
        with pytest.raises(st.TensorError):
            bridge.register_channel(*bad)
    with pytest.raises(st.TensorError):
        bridge.set_narrative_tags("missing", ["a"])
    sem = SemanticBridge.from_dense(torch.tensor([[0.9, 0.1], [0.2, 0.8], [0.5, 0.5]]))
    d = ConceptHint.from_distribution([3.0, -1.0]).as_distribution(sem)
    assert d[0] == pytest.approx(1.0) and d[1] > 0
    assert ConceptHint.from_distribution([]).as_distribution(sem) == [0.5, 0.5]
    assert sum(hint.as_distribution(sem)) == pytest.approx(1.0, abs=1e-5)


def test_language_bridges_and_trace_recorder(tmp_path):
    seq = _seq()
    rec = seq.install_trace_recorder(C.ZSpaceTraceConfig(capacity=64, max_vector_len=8))
    assert seq.plugin_names() == ["zspace_trace"]
    seq.set_backend("fftw")
    seq.register_linguistic_profile(C.DomainLinguisticProfile("membrane"))
    seq.enable_pre_discard(C.PreDiscardPolicy(0.6))
    sem = SemanticBridge.from_dense(torch.tensor([[0.9, 0.1], [0.2, 0.8], [0.5, 0.5], [0.1, 0.9]]))
    bridge = MaxwellDesireBridge().with_channel("membrane", [(0, 1.0)], tags=["tide"])
    torch.manual_seed(1)
    x = st.Tensor._wrap(torch.randn(4, 128).abs() * 0.2 + 0.05)
    agg, coh, concept, narrative, pulse = seq.forward_with_language_bridges(x, sem, bridge)
    assert agg.shape() == (4, 128) and len(concept) == 2 and sum(concept) == pytest.approx(1.0, abs=1e-4)
    assert narrative is not None and narrative.channel == "membrane" and pulse.blocks == 4
    kinds = [r["kind"] for r in rec.records()]
    assert kinds[:2] == ["BackendConfigured", "LinguisticProfileRegistered"]
    for k in ("Projected", "CoherenceMeasured", "PreDiscardApplied", "Aggregated", "SemanticWindowDerived", "SemanticDistributionDerived",
              "CanonicalConceptSelected", "MaxwellBridgeEmitted", "SemanticWindowFused", "LanguageBridged"):
        assert k in kinds
    assert kinds.index("CoherenceMeasured") < kinds.index("PreDiscardApplied") < kinds.index("Aggregated")
    aggregated = next(r for r in rec.records() if r["kind"] == "Aggregated")
    assert len(aggregated["payload"]["coherence"]) == 8                       # vectors are cut to max_vector_len
    assert aggregated["payload"]["diagnostics"]["classification_kind"] in zc.LABELS
    assert [r["step"] for r in rec.records()] == list(range(len(kinds)))
    path = tmp_path / "trace.jsonl"
    rec.write_jsonl(path)
    lines = path.read_text().splitlines()
    assert len(lines) == len(kinds) and json.loads(lines[0])["schema"] == "spiraltorch.zspace_trace"
    small = C.ZSpaceTraceRecorder(C.ZSpaceTraceConfig(capacity=2))
    for i in range(5):
        small.on_stage("LinguisticProfilesCleared", {})
    assert small.snapshot()["dropped_events"] == 3 and [r["step"] for r in small.records()] == [3, 4]
    small.clear()
    assert small.snapshot() == {"dropped_events": 0, "events": []}
    got = []
    sid = st.plugin.subscribe("ZSpaceTrace", got.append)
    pub = C.ZSpaceTraceRecorder(C.ZSpaceTraceConfig(publish_plugin_events=True))
    pub.on_stage("CanonicalConceptSelected", {"concept": "membrane", "channel": "membrane"})
    st.plugin.unsubscribe("ZSpaceTrace", sid)
    assert got and got[0]["record"]["payload"]["concept"] == "membrane"
    seq.clear_plugins()
    assert seq.plugin_names() == []
    r = C.coherence_relation_tensor([0.5, 1.0, float("nan")]).torch()
    assert r.shape == (3, 3) and r[1, 1] == 1.0 and r[0, 1] == 0.5 and r[2, 2] == 0.0
    with pytest.raises(st.TensorError):
        C.coherence_relation_tensor([])


@pytest.mark.gpu
def test_sequencer_on_gpu_matches_cpu():
    torch.manual_seed(2)
    x = torch.randn(64, 256) * 0.4
    seq = C.ZSpaceCoherenceSequencer(256, 8, -1.0, OpenCartesianTopos(-1.0, 1e-5, 10.0, 256, 1 << 20))
    out_c, coh_c, d_c = seq.forward_with_diagnostics(st.Tensor._wrap(x))
    out_g, coh_g, d_g = seq.forward_with_diagnostics(st.Tensor._wrap(x.cuda()))
    assert out_g.torch().is_cuda
    assert torch.allclose(out_g.torch().cpu(), out_c.torch(), atol=2e-5)
    assert coh_g == pytest.approx(coh_c, abs=1e-5) and d_g.dominant_channel == d_c.dominant_channel
