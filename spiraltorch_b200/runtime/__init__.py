"""Host runtime: native worker pool / rendezvous / loader bindings and the multi-trainer driver."""
from . import blackcat, golden, host
from .golden import (GoldenDropoutRecord, GoldenEpochReport, GoldenRetriever, GoldenRetrieverConfig, GoldenRuntime,
                     GoldenRuntimeConfig)
from .host import NativeRendezvous, PrefetchLoader, WorkerFailure, WorkerPool, atomic_write
