"""Registers the parts that ship with the framework."""
from .attention import GQA, TalkingAttention
from .base import register_part
from .block import OutNorm, PreNorm, Sandwich
from .embedding import Embedding, Head, PairEmbedding
from .experts import Experts
from .feedforward import MLP, ClampedGLU, SwiGLU
from .hyper import Hyper
from .latent import LatentAttention
from .norm import DynamicTanh, RMSNorm
from .parallel import ParallelBlock, SideBySide
from .position import Rope
from .recurrent import MLSTM, GatedDelta, GeneralDelta, Retention

register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("position", "rope", Rope, replace=True)
register_part("mixer", "gqa", GQA, replace=True)
register_part("mixer", "latent", LatentAttention, replace=True)
register_part("ffn", "swiglu", SwiGLU, replace=True)
register_part("ffn", "experts", Experts, replace=True)
register_part("block", "prenorm", PreNorm, replace=True)
register_part("block", "hyper", Hyper, replace=True)
register_part("embed", "table", Embedding, replace=True)
register_part("head", "linear", Head, replace=True)
register_part("mixer", "retention", Retention, replace=True)
register_part("mixer", "gated_delta", GatedDelta, replace=True)
register_part("mixer", "side_by_side", SideBySide, replace=True)
register_part("ffn", "clamped_glu", ClampedGLU, replace=True)
register_part("block", "parallel", ParallelBlock, replace=True)
register_part("embed", "pair", PairEmbedding, replace=True)
register_part("mixer", "talking", TalkingAttention, replace=True)
register_part("mixer", "mlstm", MLSTM, replace=True)
register_part("ffn", "mlp", MLP, replace=True)
register_part("block", "outnorm", OutNorm, replace=True)
register_part("norm", "dyt", DynamicTanh, replace=True)
register_part("block", "sandwich", Sandwich, replace=True)
register_part("mixer", "general_delta", GeneralDelta, replace=True)
