"""spiraltorch-b200: a Blackwell-native framework with the public API of SpiralTorch.

``import spiraltorch_b200 as st`` (or ``import spiraltorch as st``) gives ``st.Tensor``, ``st.nn``,
``st.optim``, ``st.SpiralSession``, ``st.plugin``, ``st.selfsup``, ``st.build_info()`` and
``st.describe_device()``.  CUDA work runs on hand-written sm_100a kernels (``csrc/``).
"""
from . import (advisors, api_llm, autograd, compress, config, device_caps, differential, drift_response, engine, inference, measure, distributed, hf_bridge, hf_study, hpo, kdsl, language, logic, metrics, nn, observability, optim, plugin, rec, rl, robotics, runtime, safety,
               selfsup, softlogic, telemetry, text, theory, topos, tracking, vision, zspace_coherence, zvolume)
from . import (ecosystem, elliptic, hub, inflaton, introspect, kdsl_ir, kv, macro_model, mellin, meta_narrative, microlocal, observation, psi_sync, psychoid, qr_studio, quantum_overlay, quantum_reality, sot, relativity,
               rg_flow, schrodinger, soft_learning, spiral_dynamics, stv, sync_bridge, unison, zpulse, zspace_posterior)  # noqa: E402  (network key/value client imports logic)
from .nn.io import VERSION as __version__
from .optim.amegagrad import AmegaHypergrad as Hypergrad, AmegaRealgrad as Realgrad
from .session import SpiralSession, build_info, describe_device
from .tensor import NonFiniteValue, Tensor, TensorError, set_default_device, set_finite_checks


def hypergrad(rows: int, cols: int, *, curvature: float = -1.0, learning_rate: float = 1e-2, topos=None):
    """``st.hypergrad(rows, cols, curvature=..., learning_rate=...)`` notation of the reference."""
    return Hypergrad(curvature, learning_rate, rows, cols, topos=topos)


def realgrad(rows: int, cols: int, *, learning_rate: float = 1e-2):
    return Realgrad(learning_rate, rows, cols)


def init_backend(name: str = "auto") -> str:
    """Resolve a backend label to the backend that will run (``cpu`` or ``cuda``)."""
    return SpiralSession(name).effective_backend

from .elliptic import EllipticTelemetry, EllipticWarp  # noqa: E402  (top-level names of the reference's Python surface)
from .introspect import clear_zspace_feedback, describe_zspace, softlogic_feedback, softlogic_signal, zspace_snapshot  # noqa: E402
