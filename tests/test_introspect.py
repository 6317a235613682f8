"""Z-space regions and the hub's feedback readers."""
import pytest

import spiraltorch_b200 as st
from spiraltorch_b200 import hub, introspect as I
from spiraltorch_b200.elliptic import EllipticWarp
from spiraltorch_b200.zpulse import ZScale


@pytest.fixture(autouse=True)
def clean():
    hub.reset()
    yield
    hub.reset()


def test_band_classification_and_descriptor():
    assert [I.ZSpaceSpinBand.classify(v) for v in (0.8, -0.9, 0.1)] == ["leading", "trailing", "neutral"] and I.ZSpaceSpinBand.values == ("leading", "neutral", "trailing")
    assert [I.ZSpaceRadiusBand.classify(v) for v in (0.1, 0.5, 0.9)] == ["core", "mantle", "edge"]
    sample = {"curvature_radius": 1.0, "geodesic_radius": 0.2, "normalized_radius": 0.2, "spin_alignment": 0.7, "sheet_index": 2, "sheet_count": 4,
              "topological_sector": 3}
    d = I.ZSpaceRegionDescriptor.from_elliptic(sample)
    assert d.key() == I.ZSpaceRegionKey("leading", "core") and d.label() == "spin.leading.radius.core"
    events = []
    with st.observability.observe(events.append):
        e = I.ZSpaceRegionDescriptor.from_elliptic({**sample, "spin_alignment": -0.8, "normalized_radius": 1.9})
    meta = [ev["meta"] for ev in events if ev["kind"] == "tensor_op_meta"][0]
    assert e.normalized_radius == 1.0 and meta["spin_band"] == "spin.trailing" and meta["radius_band"] == "radius.edge"
    assert meta["region_label"] == "spin.trailing.radius.edge"


def test_hub_readers():
    assert I.snapshot() is None and I.feedback() is None and I.describe() is None and I.softlogic_signal() is None and not I.clear()
    with pytest.raises(RuntimeError):
        I.describe_zspace(latest=False)
    plain = hub.SoftlogicZFeedback(psi_total=1.0, band_energy=(0.2, 0.5, 0.3), drift=0.1, z_signal=0.4, events=["a"], attributions=[("maxwell", 0.5)])
    hub.set_softlogic_z(plain)
    assert I.snapshot() is None and I.describe(feedback=True) is plain and I.describe() is None      # no elliptic record: no region
    sig = I.softlogic_signal()
    assert sig["band_energy_detail"] == {"above": 0.2, "here": 0.5, "beneath": 0.3, "total": 1.0, "drift": 0.1} and "region" not in sig and sig["scale"] is None
    tel = EllipticWarp(2.0).with_sheet_count(4).map_orientation([1.0, 1.0, 0.2])
    hub.set_softlogic_z(hub.SoftlogicZFeedback(z_signal=0.1, scale=ZScale.new(2.0), elliptic=tel.as_dict()))
    region = I.zspace_snapshot()
    assert region.sheet_count == 4 and region.key().radius == "mantle" and region.spin_alignment == pytest.approx(tel.spin_alignment)
    assert I.softlogic_signal()["region"] == region and I.softlogic_signal()["scale"] == (2.0, pytest.approx(0.6931, abs=1e-4))
    assert I.clear_zspace_feedback() and I.softlogic_feedback() is None
    assert set(I.__all__) <= set(dir(I))
