"""Psychoid meter: metric definitions, robust z-scores, CTI score, dream events (behaviour of
crates/st-core/src/telemetry/psychoid.rs)."""
import math

import pytest
import torch

from spiraltorch_b200 import psychoid as P


def _frame(i, text, logits=None, hidden=None):
    return P.PsychoidFrame(i, logits if logits is not None else [0.0, 0.0, 0.0], hidden if hidden is not None else [1.0, 0.0], text)


def test_robust_z_and_lexicon_counts():
    assert P.robust_z(5.0, [1.0] * 19) == 0.0                                    # needs 20 samples
    hist = [float(i) for i in range(21)]
    assert P.robust_z(15.0, hist) == pytest.approx((15.0 - 10.0) / (1.4826 * 5.0))
    assert P.robust_z(3.0, [2.0] * 25) == pytest.approx(1.0 / (1.4826 * 1e-6), rel=1e-3)      # MAD floor
    assert P.count_occurrences("I cannot. I CANNOT assist with that; stay safe!", P.RITUAL_STEMS) == 3
    assert P.extract_shadow_phrases("This may be harmful, so I cannot provide it") == ["i cannot", "harmful", "cannot provide"]
    m = P.motif_from_text("the hero crossed the gate on a quest")
    assert m[6] == pytest.approx(2 / 8) and m[7] == pytest.approx(1 / 8) and m[0] == 0.0


def test_metric_definitions_on_a_small_window():
    meter = P.PsychoidMeter(window=8)
    frames = [_frame(0, "Yes, indeed ", [2.0, 0.0, 0.0], [1.0, 0.0]), _frame(1, "the sacred spiral ", [0.0, 2.0, 0.0], [0.0, 1.0]),
              _frame(2, "however I cannot ", [0.0, 2.0, 0.0], [0.0, 2.0])]
    reading, events = meter.observe(P.PsychoidSample("tell me about the spiral", "Yes, indeed the sacred spiral however I cannot", frames))
    p, q = torch.softmax(torch.tensor([2.0, 0, 0]), -1), torch.softmax(torch.tensor([0.0, 2, 0]), -1)
    kl = float((p * (torch.log(p + 1e-8) - torch.log(q + 1e-8))).sum())
    assert reading.get_raw("D") == pytest.approx(kl / 2, rel=1e-5)                          # second pair is identical: KL 0
    assert reading.get_raw("C") == pytest.approx(1.0 - 0.5, rel=1e-6)                        # cosines 0 and 1
    assert reading.get_raw("K") == 0.0                     # the anchor is the first distribution the meter scores: itself
    words = 8
    assert reading.get_raw("S") == pytest.approx(2 / words + 0.01)
    assert reading.get_raw("H") == 1.0 and reading.get_raw("RR") == pytest.approx(1 / words) and reading.get_raw("RRI") == pytest.approx(1 / words)
    overlap = 2 / 8                                                                         # "the", "spiral" of the window's 8 distinct words
    assert reading.get_raw("NU") == pytest.approx(max(1 / words - 0.25 * overlap, 0.0))
    assert reading.get_raw("SE") == 1.0 and reading.get_raw("TD") == 0.0
    assert reading.get_raw("AX") == pytest.approx(0.35 * reading.get_raw("D") + 0.25 * 0.5 + 0.25 / words + 0.15 * reading.get_raw("NU"))
    assert all(v == 0.0 for v in reading.z_scores.values()) and reading.step == 1           # no history yet
    assert reading.cti == pytest.approx(P.cti_score(P.motif_from_text("tell me about the spiral Yes, indeed the sacred spiral however I cannot"),
                                                     [0.0] * 11, reading.z_scores, meter.params))
    assert reading.cti == pytest.approx(0.5) and events == []                                # zero metric vector: cosine 0
    assert meter.observe(P.PsychoidSample()) is None and meter.step == 2
    r2, _ = meter.observe(P.PsychoidSample("p", "g", [_frame(3, "we can classify ", [2.0, 0.0, 0.0])]))
    assert r2.get_raw("TD") == 1.0 and r2.get_raw("RRI") == pytest.approx(1 / 11 - 1 / 8)
    assert r2.get_raw("K") == pytest.approx(float((p * (torch.log(p + 1e-8) - torch.log(q + 1e-8))).sum()), rel=1e-5)   # KL(now || anchor)


def test_cti_score_and_events():
    params = P.CTIParams()
    f = [1.0] + [0.0] * 11
    z = {k: 0.0 for k in P.METRIC_KEYS}
    m = [1.0] + [0.0] * 10
    base = P.cti_score(f, m, z, params)
    assert base == pytest.approx(1 / (1 + math.exp(-0.75)))                                  # aligned motif and metric vectors
    z["RRI"], z["AX"] = 2.0, -3.0                                                            # negative z-scores are clipped
    assert P.cti_score(f, m, z, params) == pytest.approx(1 / (1 + math.exp(-(0.75 + 0.9))))
    z["AX"] = 1.0
    assert P.cti_score(f, m, z, params) == pytest.approx(1 / (1 + math.exp(-(0.75 + 0.9 - 0.35))))
    replay = P.dream_replay(["i cannot", "safety policy", "harmful"])
    assert replay.symbols == ["threshold", "bridge", "lantern"] and "bridge" in replay.diary and '"i cannot, safety policy"' in replay.diary
    assert P.dream_replay([]) is None and P.dream_replay(["i cannot"]).diary == P.dream_replay(["i cannot"]).diary     # deterministic
    # a stream that turns to refusal boilerplate after a calm history raises a dream-pass event
    meter = P.PsychoidMeter(window=4, params=P.CTIParams(tau2=2.0))          # export branch out of reach: the pass branch decides
    torch.manual_seed(0)
    events = []
    for i in range(40):
        text = "plain words here " if i < 30 else "As an AI I cannot do that, stay safe. "
        out = meter.observe(P.PsychoidSample("question", text, [_frame(i, text, torch.randn(5) * 0.01, torch.randn(4))]))
        events += out[1]
    assert events and events[0].kind == "dream_pass" and events[0].step > 30 and events[0].cti > 0.62
    # with the default thresholds the same stream lands in the export branch, which needs symbol words and a calm axis
    strict = P.PsychoidMeter(window=4)
    torch.manual_seed(0)
    kinds = []
    for i in range(40):
        text = "plain words here " if i < 30 else "I cannot, stay safe: the spiral bridge and the lantern. "
        kinds += [e.kind for e in strict.observe(P.PsychoidSample("question", text, [_frame(i, text, torch.randn(5) * 0.01, torch.randn(4))]))[1]]
    assert set(kinds) <= {"dream_export"}
