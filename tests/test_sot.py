"""SoT-3D-phi spiral plans: pacing, packing, geometry, tensor exports, biome deposit."""
import math

import pytest
import torch

import spiraltorch_b200 as st
from spiraltorch_b200 import sot


def test_pacing_and_packing():
    assert sot.fibonacci_pacing(12) == [1, 1, 2, 3, 5] and sot.fibonacci_pacing(10) == [1, 1, 2, 3, 3] and sot.fibonacci_pacing(0) == []
    # the admissible chunk closest to half of what remains; the larger one on ties
    assert sot.pack_tribonacci_chunks(13) == [7, 4, 1, 1] and sot.pack_tribonacci_chunks(5) == [2, 2, 1] and sot.pack_tribonacci_chunks(0) == []
    assert sot.pack_tetranacci_chunks(16) == [8, 4, 2, 1, 1] and sot.pack_tetranacci_chunks(3) == [2, 1]
    for n in range(1, 60):
        assert sum(sot.pack_tribonacci_chunks(n)) == n and sum(sot.pack_tetranacci_chunks(n)) == n
    assert sot.golden_angle() == pytest.approx(math.pi * (3 - math.sqrt(5))) and sot.golden_ratio() == pytest.approx((1 + math.sqrt(5)) / 2)
    assert set(sot.__all__) <= set(dir(sot))


def test_plan_geometry_and_grouping():
    plan = sot.generate_plan(12, base_radius=2.0, radial_growth=0.1, base_height=1.0, meso_gain=0.2, micro_gain=0.05)
    steps = plan.steps()
    assert len(steps) == 12 and [m.length for m in plan.macro_summaries()] == [1, 1, 2, 3, 5] and plan.macro_summaries()[4].ideal_length == 5
    s = steps[7]                                                       # first step of the fifth orbit (start 7, length 5)
    assert (s.macro_index, s.macro_position, s.macro_length, s.macro_phase) == (4, 0, 5, 0.0)
    assert s.angle == pytest.approx(sot.GOLDEN_ANGLE * 7) and s.radius == pytest.approx(2.0 * math.exp(0.7))
    assert (s.x, s.y) == pytest.approx((s.radius * math.cos(s.angle), s.radius * math.sin(s.angle)))
    assert s.curvature == pytest.approx(math.sqrt(1.01) / s.radius)
    # heights: each orbit climbs base_height / phi^k in equal steps; the meso / micro phases wobble around the track
    track = 1.0 + 1 / sot.GOLDEN_RATIO + 1 / sot.GOLDEN_RATIO ** 2 + 1 / sot.GOLDEN_RATIO ** 3 + (1 / sot.GOLDEN_RATIO ** 4) / 5
    assert s.z_track == pytest.approx(track) and s.height == pytest.approx(track + 0.2 * (s.meso_phase - 0.5) + 0.05 * (s.micro_phase - 0.5))
    assert steps[-1].macro_reflection and steps[-1].meso_reflection and steps[-1].micro_reflection and not steps[7].macro_reflection
    assert [m.reflection_step for m in plan.macro_summaries()] == [0, 1, 3, 6, 11]
    assert plan.macro_summaries()[2].height_gain == pytest.approx(1 / sot.GOLDEN_RATIO ** 2)
    assert plan.macro_summaries()[2].mean_curvature == pytest.approx((steps[2].curvature + steps[3].curvature) / 2)
    # roles cycle with the global chunk counters
    assert [st_.meso_role for st_ in steps[:4]] == ["explore", "structure", "verify", "verify"] or steps[0].meso_role == "explore"
    assert all(st_.meso_role == sot.MESO_ROLES[st_.meso_index % 3] and st_.micro_role == sot.MICRO_ROLES[st_.micro_index % 4] for st_ in steps)
    assert (0, "micro") in plan.reflection_points() and (11, "macro") in plan.reflection_points()
    assert plan.polyline[3] == steps[3].position and steps[3].as_dict()["index"] == 3 and "steps=12" in repr(plan)
    empty = sot.generate_plan(0)
    assert empty.steps() == [] and empty.as_tensor().shape() == (0, 3) and empty.macro_summary_tensor().shape() == (0, 6)
    with pytest.raises(ValueError):
        sot.generate_plan(-1)


def test_tensor_exports_and_seeded_rotation():
    plan = sot.generate_plan(20)
    steps = plan.steps()
    pos, feat = plan.as_tensor().torch(), plan.feature_tensor().torch()
    assert pos.shape == (20, 3) and feat.shape == (20, 9)
    assert torch.allclose(pos[5], torch.tensor([steps[5].x, steps[5].y, steps[5].height], dtype=torch.float32))
    assert feat[5, 0] == pytest.approx(steps[5].radius) and feat[5, 7] == pytest.approx(0.2) and feat[5, 8] == pytest.approx(0.05)
    roles, refl, macro = plan.role_tensor().torch(), plan.reflection_tensor().torch(), plan.macro_summary_tensor().torch()
    assert roles.shape == (20, 2) and refl.shape == (20, 3) and macro.shape == (len(plan.macro_summaries()), 6)
    assert refl[:, 0].sum() == len(plan.macro_summaries()) and macro[-1, 5] == 19 and roles[:, 1].max() <= 3
    assert plan.biome_tensor().shape() == (20, 16) and plan.biome_tensor(False, False).shape() == (20, 11) and plan.biome_tensor(True, False).shape() == (20, 14)
    a, b, c = sot.generate_plan(20, seed=7), sot.generate_plan(20, seed=7), sot.generate_plan(20, seed=8)
    assert a.steps()[3].angle == b.steps()[3].angle != c.steps()[3].angle
    off = a.steps()[0].angle
    assert 0 <= off < 2 * math.pi and a.steps()[4].angle == pytest.approx(sot.GOLDEN_ANGLE * 4 + off)
    assert a.steps()[4].radius == plan.steps()[4].radius and a.steps()[4].height == plan.steps()[4].height
    assert a.steps()[4].x == pytest.approx(a.steps()[4].radius * math.cos(a.steps()[4].angle))


def test_biome_deposit():
    topos = st.topos.OpenCartesianTopos(-1.0, 1e-6, 1e6, 16, 1 << 16)
    plan = sot.generate_plan(9, meso_gain=0.3, micro_gain=0.1)
    biome = plan.grow_biome(topos, "route")
    assert len(biome) == 1 and biome.total_weight() == pytest.approx(1.4) and biome.shape() == (9, 16)
    plan.infuse_biome(biome, None, include_reflections=True, include_roles=True)
    assert len(biome) == 2 and biome.total_weight() == pytest.approx(2.8)
