"""Layers put together from parts: mixer, feed-forward, norm, position encoding, block arrangement."""
from .base import (Addend, BuildContext, FeedForward, Mixer, Norm, Part, PositionEncoding, make_part, register_part,
                   unregister_part)
from .context import CacheView, GroupStep, ResidualStream, StepContext, Workspace
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from . import norm, rotary, embedding, attention, feed_forward, block  # noqa: F401  (register the parts)
from .model import DecoderModel

__all__ = [
    "Addend", "BuildContext", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "make_part",
    "register_part", "unregister_part", "CacheView", "GroupStep", "ResidualStream", "StepContext", "Workspace",
    "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "DecoderModel",
]
