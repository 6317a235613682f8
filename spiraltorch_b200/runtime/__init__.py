"""Host runtime: native worker pool / rendezvous / loader bindings and the multi-trainer driver."""
from . import autopilot, blackcat, golden, host, trainer_external, zspace_optimizer
from .golden import (GoldenDropoutRecord, GoldenEpochReport, GoldenRetriever, GoldenRetrieverConfig, GoldenRuntime,
                     GoldenRuntimeConfig)
from .host import NativeRendezvous, PrefetchLoader, WorkerFailure, WorkerPool, atomic_write
from .zspace_optimizer import ZSpaceMetaOptimizer
