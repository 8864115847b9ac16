"""The parts a decoder is assembled from, and their registration under their kind names."""
from .. import registry
from .base import (FeedForward, KVRequest, KVStateRequest, Mixer, Norm, Part, PositionEncoding, Runtime, StateRequest,
                   TensorDecl)
from .attention import Attention
from .block import PreNormBlock
from .delta_rule import DeltaRule
from .dense_ff import ClampedGLU, ReluSquared
from .diff_attention import DiffAttention
from .latent_attention import LatentAttention
from .postnorm import PostNormBlock
from .gated_attention import GatedAttention
from .hyper import HyperBlock
from .linear_state import DecayState, MatrixMemory
from .moe import MoE
from .norm import RMSNorm
from .reinject import Reinject
from .rope import NoPosition, PairRotaryEmbedding, RotaryEmbedding
from .sigmoid_attention import SigmoidAttention
from .swiglu import SwiGLU

registry.register_norm("rmsnorm", RMSNorm)
registry.register_position("rope", RotaryEmbedding)
registry.register_position("rope_pairs", PairRotaryEmbedding)
registry.register_position("none", NoPosition)
registry.register_mixer("attention", Attention)
registry.register_mixer("gated_attention", GatedAttention)
registry.register_mixer("gla", DecayState)
registry.register_mixer("mlstm", MatrixMemory)
registry.register_mixer("sigmoid_attention", SigmoidAttention)
registry.register_mixer("delta_rule", DeltaRule)
registry.register_mixer("diff_attention", DiffAttention)
registry.register_mixer("latent_attention", LatentAttention)
registry.register_feed_forward("swiglu", SwiGLU)
registry.register_feed_forward("relu2_ff", ReluSquared)
registry.register_feed_forward("glu_clamp", ClampedGLU)
registry.register_feed_forward("moe", MoE)
registry.register_block("prenorm", PreNormBlock)
registry.register_block("hyper", HyperBlock)
registry.register_block("postnorm", PostNormBlock)
registry.register_junction("reinject", Reinject)

__all__ = ["ClampedGLU", "DiffAttention", "LatentAttention", "PostNormBlock", "ReluSquared", "Attention", "DecayState", "DeltaRule", "FeedForward", "GatedAttention", "HyperBlock", "KVStateRequest", "MatrixMemory", "MoE", "SigmoidAttention", "PairRotaryEmbedding", "KVRequest", "Mixer", "NoPosition", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "Reinject", "RMSNorm", "RotaryEmbedding", "Runtime", "StateRequest", "SwiGLU", "TensorDecl"]
