"""Drop-in name for users of the reference package: ``import spiraltorch as st``.

Everything is provided by :mod:`spiraltorch_b200`; this module only aliases it, including the
sub-modules (``spiraltorch.nn``, ``spiraltorch.optim``, ...).
"""
import sys as _sys

import spiraltorch_b200 as _impl
from spiraltorch_b200 import *  # noqa: F401,F403
from spiraltorch_b200 import (SpiralSession, Tensor, build_info, config, describe_device, distributed, hypergrad,
                              init_backend, nn, optim, plugin, realgrad, selfsup)

__version__ = _impl.__version__
for _name in ("nn", "optim", "plugin", "selfsup", "config", "distributed", "autograd", "compress", "engine", "measure", "hpo", "kdsl", "language", "text", "metrics", "rec", "rl",
              "robotics", "runtime", "safety", "softlogic", "telemetry"):
    _sys.modules[f"{__name__}.{_name}"] = getattr(_impl, _name)
