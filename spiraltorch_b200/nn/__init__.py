"""``spiraltorch.nn``: modules, losses, trainer, data and weight files of the public API."""
from .amp import (AutocastGuard, CoherenceSignal, CurvatureDecision, CurvatureScheduler, GradScaler, OptimizerMode,
                  SpectralAdjustment, SpectralLearningRatePolicy, SpectralLrAdapter, WarmupCosineScheduler,
                  ZSpaceParameterOptimizer, autocast_enabled)
from .data import DataLoader, DataLoaderIter, Dataset, from_samples
from .io import load, load_bincode, load_json, save, save_bincode, save_json
from .losses import (CategoricalCrossEntropy, ContrastiveLoss, CrossEntropy, FocalLoss, HyperbolicCrossEntropy,
                     Loss, MeanSquaredError, SoftmaxCrossEntropy, TripletLoss)
from .modules import (BatchNorm1d, Dropout, Embedding, FeatureReorder2d, Gelu, Identity, LayerNorm, Linear,
                      LoraLinear, Lstm, Module, NonLiner, Parameter, Pool2d, Relu, Scaler, Sequential, SpiralRnn,
                      WaveGate, WaveRnn, ZConv, ZPooling, ZSpaceBatchNorm1d, ZSpaceCoherenceScan,
                      ZSpaceCoherenceWaveBlock, ZSpaceLayerNorm, ZSpaceMixer, ZSpaceSoftmax, conv_output_shape,
                      pool_output_shape, reorder_feature_tensor, reorder_feature_tensor_3d)
from .trainer import EpochStats, ModuleTrainer, RoundtableConfig, RoundtableSchedule, SoftLogicConfig, StepMetrics
from . import amp, coherence, conv, fields, gnn, graph, lightning, roundtable, zrba, zspace
from .graph import GraphedTrainStep
from .zrelativity import ZRelativityModule
py_is_swap_invariant = None  # bound below, once the coherence names are imported
from .roundtable import DistConfig, MetaConductor, MetaSummary, RoundtableNode
from .conv import AvgPool2d, Conv2d, Conv3d, Conv4d, Conv6da, MaxPool2d, WaveScan, ZConv6DA
from .fields import (ContinuousWavelet, Conv1d, DynamicHamiltonJacobiField, DynamicKleinGordonField,
                     DynamicSchrodingerField, ToposResonator, ZRelativity, ZSpaceProjector)
from .gnn import (GraphBatch, GraphContext, GraphReadout, NeighborhoodAggregation, RoundtableBandInfluence, RoundtableBandSignal,
                  RoundtableGnnBridge, ZSpaceGraphBatchRegressor,
                  ZSpaceGraphConvolution, ZSpaceGraphNetwork, ZSpaceGraphRegressor)
from .lightning import (InfoNCELoss, LightningConfig, LightningReport, LightningStage, SelfSupStage, SpiralLightning)
from .zrba import (BetaGate, BetaGateConfig, BetaGateSample, CovHead, CovHeadTelemetry, ReliabilityBin,
                   SpectralFeatureSample, ZCov, ZRBA, ZRBAConfig, ZRBAMetrics, ZRBATelemetry, ZTelemetryBundle)
from .zspace import (ArdParameters, LanguageWaveEncoder, MellinBasis, ZFrame, ZIndex, ZMetricWeights, ZRBFAttention,
                     ZSpaceTextVae, ZSpaceVae, ZSpaceVaeBatchStats, ZSpaceVaeState, ZSpaceVaeStats, ZTensor)
from .coherence import (CoherenceBackend, CoherenceChannelReport, CoherenceDiagnostics, CoherenceEngine, CoherenceObservation,
                        CoherenceSignature, DomainLinguisticProfile, LinguisticChannelReport, LinguisticContour,
                        PreDiscardPolicy, PreDiscardRegulator, PreDiscardSnapshot, PreDiscardTelemetry,
                        ZSpaceCoherenceSequencer, ZSpaceTraceConfig, ZSpaceTraceRecorder, coherence_relation_tensor,
                        is_swap_invariant)
from ..language import ConceptHint, MaxwellDesireBridge, NarrativeHint, NarrativeSummary
from ..desire_pipeline import (DesirePipeline, DesirePsiBridge, DesirePsiEvent, DesirePsiSummary, DesireRoundtableBridge,
                               DesireTelemetryBundle, DesireTrainerBridge)

NnModuleTrainer = ModuleTrainer          # the binding registers the trainer under both names
from ..runtime.golden import GoldenRetriever  # noqa: E402  (multi-trainer lives with the host runtime)

py_is_swap_invariant = is_swap_invariant          # the name the reference's binding registers (bindings/st-py/src/nn.rs:80)
