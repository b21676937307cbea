from .base import (PartSpec, KVSpec, StateSpec, Runtime, StepContext, UnitCache, Part, Norm, PositionEncoding,
                   Mixer, FeedForward, Block, StreamStep, ScaledSum)
from .registry import (register_mixer, register_feed_forward, register_norm, register_position, register_block,
                       register_embedding, register_head, register_stream_step, build_part, kinds)
from . import norm, rotary, attention, latent_attention, recurrent, composite, mlp, moe, block, embedding  # noqa: F401  (register the built-in kinds)

__all__ = ["PartSpec", "KVSpec", "StateSpec", "Runtime", "StepContext", "UnitCache", "Part", "Norm",
           "PositionEncoding", "Mixer", "FeedForward", "Block", "StreamStep", "ScaledSum", "register_mixer", "register_feed_forward",
           "register_norm", "register_position", "register_block", "register_embedding", "register_head",
           "register_stream_step", "build_part", "kinds"]
