from .spec import ClampedGLUSpec, DiffAttentionSpec, LatentAttentionSpec, PostNormLayerSpec, ReluSquaredSpec
from .spec import (AttentionSpec, DecayStateSpec, DeltaRuleSpec, EmbeddingSpec, GatedAttentionSpec, HeadSpec, HyperLayerSpec,
                   LayerSpec, MatrixMemorySpec, MoESpec, ModelSpec, NoPositionSpec, PairRotarySpec, RMSNormSpec, ReinjectSpec, RotarySpec,
                   ScheduleEntry, SigmoidAttentionSpec, SwiGLUSpec, default_schedule)
from .qwen3 import ConfigError, Qwen3Config
from .pugalix import PugalixConfig
from .vepitar import VepitarConfig
from .kalonex import KalonexConfig
from .kimilix import KimilixConfig

__all__ = ["AttentionSpec", "DecayStateSpec", "DeltaRuleSpec", "EmbeddingSpec", "GatedAttentionSpec", "HeadSpec", "HyperLayerSpec",
           "LayerSpec", "MatrixMemorySpec", "MoESpec", "ModelSpec", "NoPositionSpec", "PairRotarySpec", "RMSNormSpec", "ReinjectSpec", "RotarySpec",
           "ScheduleEntry", "SigmoidAttentionSpec", "SwiGLUSpec", "default_schedule", "ConfigError", "Qwen3Config", "PugalixConfig",
           "VepitarConfig", "KalonexConfig", "KimilixConfig", "ClampedGLUSpec", "DiffAttentionSpec", "LatentAttentionSpec",
           "PostNormLayerSpec", "ReluSquaredSpec"]
