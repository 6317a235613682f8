"""``spiraltorch.optim``: Amegagrad tapes and the flat fused optimizers."""
from .amegagrad import (AmegaHypergrad, AmegaRealgrad, Amegagrad, DesireGradientControl, Topos, amegagrad)
from .flat import FlatAdamW, FlatSGD

Hypergrad = AmegaHypergrad
Realgrad = AmegaRealgrad
