"""Parts a model is put together from, and their registries."""
from .registry import CATEGORIES, part_factory, register_part, registered
from .options import KernelOptions
from .runtime import Runtime, StepContext
from . import norms, positions, mixers, feed_forward, arrangement, ends  # register the built-in kinds
from .mixers import AttentionMixer, PagedBinding, ShortConvMixer, StateBinding
from .norms import RmsNorm
from .positions import SplitHalfRope
from .feed_forward import SwiGluFeedForward
from .arrangement import PreNormResidual
from .ends import EmbeddingInput, NormHeadOutput

__all__ = ["CATEGORIES", "part_factory", "register_part", "registered", "KernelOptions", "Runtime", "StepContext",
           "AttentionMixer", "PagedBinding", "ShortConvMixer", "StateBinding", "RmsNorm", "SplitHalfRope",
           "SwiGluFeedForward", "PreNormResidual", "EmbeddingInput", "NormHeadOutput"]
