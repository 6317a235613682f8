"""Drift-response golden values (parity: crates/spiral-safety/src/drift_response.rs unit tests)."""
import math

from spiraltorch_b200.drift_response import (AnalysisOptions, DirectionQuery, DirectionalAxis, FrameState, WordState,
                                             aggregate_penalty, analyse_word, default_thresholds, existence_load,
                                             frame_summary, trainer_penalty)


def normative_word() -> WordState:
    axes = {"metaphor": DirectionalAxis([0.08], [0.12], [0.18], [0.0], [0.0], [0.0]),
            "definition_break": DirectionalAxis([-0.2], [0.9], [0.6], [0.1], [0.5], [0.05])}
    frame = FrameState(phi=0.65, c=0.9, s=0.8, a_den=-0.05, a_con=0.2, b_den=0.4, b_con=0.8, kappa=0.35,
                       directional_axes=axes)
    return WordState("AI", 0.72, {"Normative": frame}, timing_signal=1.4)


def test_existence_load_matches_reference():
    assert abs(existence_load(normative_word()) - 0.5489586) < 1e-6


def test_analyse_word_flags_radius_and_penalty():
    m = analyse_word(normative_word(), default_thresholds())
    assert abs(m.frame_hazards["Normative"] - 0.72005105) < 1e-6
    assert abs(m.safe_radii["Normative"] - 0.15151516) < 1e-6
    assert m.strict_mode and m.chi == 0
    s = m.frame_signatures["Normative"]
    assert abs(s.value_slope - 0.1125) < 1e-6 and abs(s.risk_slope - 0.528) < 1e-6 and abs(s.net_slope + 0.4155) < 1e-6
    mult = math.exp(0.72 * 0.65 * 1.4)
    assert abs(s.hazard_multiplier - mult) < 1e-6 and abs(s.timing_elasticity - mult * 0.72 * 0.65) < 1e-6
    assert s.safe_radius == m.safe_radii["Normative"] and s.tipping_radius is None
    assert abs(trainer_penalty(m) - 0.98922855) < 1e-6
    assert abs(aggregate_penalty([m, m], 0.2) - 2 * 0.98922855) < 1e-6
    assert abs(frame_summary(m)["Normative"] - 0.72005105 / 0.15151516) < 1e-4


def test_directional_queries_drive_extra_penalty():
    word, th = normative_word(), default_thresholds()
    opts = AnalysisOptions(direction_queries={"Normative": [DirectionQuery("metaphor", [1.0], "metaphor"),
                                                            DirectionQuery("definition_break", [1.0]),
                                                            DirectionQuery("absent", [1.0])]})
    m = analyse_word(word, th, opts)
    d = m.direction_signatures["Normative"]
    assert set(d) == {"metaphor", "definition_break"}
    assert d["definition_break"].safe_radius < 0.2 and d["definition_break"].hazard > d["metaphor"].hazard
    assert trainer_penalty(m, 0.2) > trainer_penalty(analyse_word(word, th))
    # a weight vector of the wrong length falls back to the frame's own mixes
    fb = analyse_word(word, th, AnalysisOptions(direction_queries={"Normative": [DirectionQuery("metaphor", [1.0, 2.0])]}))
    assert abs(fb.direction_signatures["Normative"]["metaphor"].value_slope - 0.1125) < 1e-9


def test_hazard_cut_and_quiet_word():
    quiet = WordState("tree", 0.1, {"Physical": FrameState(phi=0.1, c=0.5, s=0.1, a_den=0.5, a_con=0.5, b_den=0.1,
                                                         b_con=0.1, kappa=0.2)})
    m = analyse_word(quiet)
    assert m.frame_hazards["Physical"] == 0.0 and not m.strict_mode and trainer_penalty(m) == 0.0
    loud = analyse_word(normative_word(), default_thresholds(), AnalysisOptions(hazard_cut=0.5))
    assert loud.chi == 1
