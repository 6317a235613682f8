"""Concept diffusion and free-energy scoring (parity: crates/st-core/src/inference/concept_diffusion.rs
and crates/st-core/src/heur/free_energy.rs unit tests)."""
import math

import pytest
import torch

from spiraltorch_b200.inference import (BandEnergy, ConceptDiffusionConfig, ConceptDiffusionError,
                                        ConceptDiffusionObservation, FreeEnergyConfig, FreeEnergyError,
                                        FreeEnergyObservation, apply_concept_diffusion,
                                        blend_concept_diffusion_observation, compare_fisher_rao, evaluate_free_energy,
                                        score_with_free_energy)

PAIR = [[0.0, 1.0], [1.0, 0.0]]


def test_heat_flow_moves_a_peak_toward_uniformity():
    o = apply_concept_diffusion(["left", "right"], [1.0, 0.0], PAIR, config=ConceptDiffusionConfig(0.25))
    assert o.next_state.tolist() == [0.75, 0.25]
    e = o.effects
    assert e.entropy_after_diffusion > e.entropy_after_bias and e.dirichlet_energy_after < e.dirichlet_energy_before
    assert (e.substeps, e.edge_count, o.conductivity_source) == (1, 1, "uniform")
    again = apply_concept_diffusion(["left", "right"], [0.75, 0.25], PAIR, config=ConceptDiffusionConfig(0.25))
    assert again.next_state[0] < 0.75 and again.next_state[1] > 0.25


def test_z_bias_tilts_and_observation_blends():
    o = apply_concept_diffusion(["a", "b"], [0.5, 0.5], [[0, 0], [0, 0]], z_bias=[0.0, 2.0], config=ConceptDiffusionConfig(0.5))
    assert o.next_state[1] > 0.5 and o.effects.z_bias_applied and not o.effects.diffusion_applied
    assert abs(float(o.next_state[1]) - math.e / (1 + math.e)) < 1e-12
    b = blend_concept_diffusion_observation([0.8, 0.2], ConceptDiffusionObservation([0.2, 0.8], 0.25))
    assert abs(float(b[0]) - 0.65) < 1e-12 and abs(float(b.sum()) - 1.0) < 1e-12
    with pytest.raises(ConceptDiffusionError):
        blend_concept_diffusion_observation([0.8, 0.2], ConceptDiffusionObservation([0.2, 0.8], 1.5))


def test_cfl_substeps_and_closed_edges():
    o = apply_concept_diffusion(["l", "r"], [1.0, 0.0], PAIR, config=ConceptDiffusionConfig(2.0))
    assert o.effects.substeps == 3 and bool((o.next_state >= 0).all()) and abs(float(o.next_state.sum()) - 1) < 1e-12
    aff = [[0, 1, 1], [1, 0, 0], [1, 0, 0]]
    closed = [[1, 1, 0], [1, 1, 1], [0, 1, 1]]
    o = apply_concept_diffusion(["source", "open", "closed"], [1.0, 0.0, 0.0], aff, diffusion_tensor=closed,
                                config=ConceptDiffusionConfig(0.25))
    assert o.next_state[1] > 0 and o.next_state[2] == 0 and o.conductivity_source == "request"
    with pytest.raises(ConceptDiffusionError, match="budget"):
        apply_concept_diffusion(["l", "r"], [1.0, 0.0], PAIR, config=ConceptDiffusionConfig(2.0, max_substeps=2))


def test_request_validation():
    for kw in (dict(state=[0.7, 0.7]), dict(state=[1.0, math.nan]), dict(affinity=[[0, 1], [2, 0]]),
               dict(affinity=[[0, -1], [-1, 0]]), dict(tags=["x", "x"]), dict(z_bias=[1.0])):
        args = dict(tags=["l", "r"], state=[1.0, 0.0], affinity=PAIR)
        args.update(kw)
        with pytest.raises(ConceptDiffusionError):
            apply_concept_diffusion(**args)
    with pytest.raises(ConceptDiffusionError):
        ConceptDiffusionConfig(-1.0)
    fr = compare_fisher_rao([0.5, 0.5], [0.5, 0.5])
    assert fr.distance < 1e-7 and abs(compare_fisher_rao([1.0, 0.0], [0.0, 1.0]).distance - math.pi) < 1e-12


def _obs():
    return FreeEnergyObservation(0.8, 0.5, 12.0, 256.0, 0.05, 0.4, 0.1, BandEnergy(0.6, 0.3, 0.1))


def test_free_energy_decomposition_and_unit_invariance():
    r = evaluate_free_energy(_obs())
    c = r.components
    assert abs(r.free_energy - (c["observed_energy"] + c["band_potential"] + c["relative_entropy"])) < 1e-14
    assert r.utility == -r.free_energy and 0 <= r.acceptance_probability <= 1
    assert abs(c["observed_energy"] - (-0.3 + 0.5 * 1.2 + 0.3 * 0.25 + 0.2 * 0.05 + 0.1)) < 1e-12
    o = _obs()
    o.step_time_ms *= 1000
    o.memory_mb *= 1024
    scaled = evaluate_free_energy(o, FreeEnergyConfig(step_time_scale_ms=10_000.0, memory_scale_mb=1024.0 * 1024.0))
    assert abs(scaled.free_energy - r.free_energy) < 1e-12


def test_free_energy_prior_cases_and_score():
    cfg = FreeEnergyConfig(prior=(0.5, 0.3, 0.2))
    r = evaluate_free_energy(FreeEnergyObservation(band=BandEnergy(5.0, 3.0, 2.0)), cfg)
    assert abs(r.distribution["kl_divergence"]) < 1e-14 and abs(r.components["band_potential"]) < 1e-14
    z = evaluate_free_energy(FreeEnergyObservation(), cfg)
    assert z.distribution["status"] == "prior_zero_mass" and abs(z.distribution["above"] - 0.5) < 1e-15
    tiny = evaluate_free_energy(FreeEnergyObservation(band=BandEnergy(1.19e-7 / 4, 1.19e-7 / 8, 0.0)))
    assert tiny.distribution["status"] == "prior_zero_mass"
    with pytest.raises(FreeEnergyError):
        evaluate_free_energy(FreeEnergyObservation(step_time_ms=-1.0))
    with pytest.raises(FreeEnergyError):
        evaluate_free_energy(_obs(), FreeEnergyConfig(loss_scale=0.0))
    good = score_with_free_energy(1.0, 0.5, 10.0, 100.0, 0.0, BandEnergy(1, 0, 0), 0.2, 0.1)
    bad = score_with_free_energy(1.0, 0.9, 10.0, 100.0, 0.0, BandEnergy(0, 0, 1), 0.2, 0.1)
    assert good > bad
    assert abs(good - (0.5 - 0.025 - 0.1 - 0.02 + 0.1)) < 1e-12
    assert score_with_free_energy(1.0, 0.5, 10.0, 100.0, 0.0, BandEnergy(1, 0, 0), 0.2, -1.0) == -math.inf


def test_zspace_softmax_projection_and_entropy_target():
    from spiraltorch_b200.inference import (ZSpaceGenerationControlError, ZSpaceSoftmaxConfig, project_zspace_softmax,
                                            zspace_entropy)
    logits = [2.0, 1.0, 0.0]
    p = project_zspace_softmax(logits, ZSpaceSoftmaxConfig(-4.0, 2.0))
    assert abs(p.base_scale - 1.0) < 1e-12 and not p.adaptive_temperature
    assert torch.allclose(p.probabilities, torch.softmax(torch.tensor(logits, dtype=torch.float64), -1))
    hot = project_zspace_softmax(logits, ZSpaceSoftmaxConfig(-4.0, 2.0, entropy_target=1.09))
    assert hot.adaptive_temperature and hot.effective_temperature > 2.0 and hot.entropy > p.entropy
    assert hot.temperature_gradient_active
    cold = project_zspace_softmax(logits, ZSpaceSoftmaxConfig(-4.0, 2.0, entropy_target=0.0, entropy_gain=10.0))
    assert cold.effective_temperature == 0.5 and not cold.temperature_gradient_active     # adjust clamped to 0.25
    assert abs(zspace_entropy([0.5, 0.5]) - math.log(2)) < 1e-12
    for bad in ((0.5, 1.0), (-1.0, 0.0)):
        with pytest.raises(ZSpaceGenerationControlError):
            ZSpaceSoftmaxConfig(*bad)
    with pytest.raises(ZSpaceGenerationControlError):
        project_zspace_softmax([math.nan], ZSpaceSoftmaxConfig(-1.0, 1.0))


def test_generation_control_represses_repeats_and_ngrams():
    from spiraltorch_b200.inference import (ZSpaceGenerationControlConfig, ZSpaceGenerationControlError,
                                            apply_zspace_generation_control)
    out = apply_zspace_generation_control([3.0, 2.9, 0.0], [7, 8, 9], [1, 7, 7])
    assert out.repression_penalties.tolist() == [2.5, 0.0, 0.0] and out.before_top_token == 7 and out.after_top_token == 8
    assert out.top_changed and out.repressed_token_count == 1 and abs(float(out.probabilities.sum()) - 1) < 1e-12
    assert torch.allclose(out.log_probabilities.exp(), out.probabilities)
    # the window bounds what is counted
    short = apply_zspace_generation_control([1.0], [7], [7, 7, 7, 1], ZSpaceGenerationControlConfig(repression_window=2))
    assert short.repression_penalties.tolist() == [1.0]
    # "1 2 3 ... 1 2" -> completing with 3 is an n-gram repeat; decay weights older matches less
    cfg = ZSpaceGenerationControlConfig(repression_strength=0.0, last_token_repression=0.0, ngram_size=3,
                                        ngram_repression_strength=2.0, ngram_decay=0.5)
    ng = apply_zspace_generation_control([1.0, 1.0], [3, 4], [1, 2, 3, 5, 1, 2, 3, 1, 2], cfg)
    assert ng.ngram_repression_penalties.tolist() == [2.0 * (0.5 ** 2 + 0.5 ** 6), 0.0] and ng.after_top_token == 4
    with pytest.raises(ZSpaceGenerationControlError, match="mismatch"):
        apply_zspace_generation_control([1.0, 2.0], [1], [])
    with pytest.raises(ZSpaceGenerationControlError):
        apply_zspace_generation_control([1.0], [1], [], ZSpaceGenerationControlConfig(ngram_decay=0.0))
