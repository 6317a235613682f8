"""Distributed training surface: rendezvous, training devices and the error vocabulary."""
from .device import (CpuDevice, DistributedDevice, MetricReduce, NativeDistributedDevice, ProcessGroupDevice,
                     TrainingDevice)
from .rendezvous import (BufferLengthMismatch, CollectiveTimeout, DistributedError, DuplicateContribution,
                         DuplicateRank, EmptyWorldSize, NonFiniteInput, NonFiniteReduction, ParticipantLeft,
                         PeerTensorFailure, RankOutOfBounds, UnknownRank, WorldSizeMismatch, join)
from .arena import (AgentConfig, AmebaAutograd, AutogradError, CollectiveArena, CollectiveError,
                    CollectiveExecutionReport, DistributedTrainer, DistributedTrainerError)
from . import lanes
