from . import (attention, block, embedding, head_normed_attention, hyper, latent_attention, linear_state, mamba2, mlp, mlstm, moe, norm,
               normed_attention, parallel, rope, sink_attention, token_side)  # noqa: F401  (registers the built-in parts)
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, WeightSpec
from .registry import lookup, register, registered, unregister
from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "WeightSpec",
           "lookup", "register", "registered", "unregister", "ExtraPart", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry"]
