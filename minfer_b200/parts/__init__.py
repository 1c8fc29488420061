"""The parts that ship with the library, registered under their kinds."""
from ..registry import register_part
from .attention import Attention
from .base import (Block, CacheRequest, CacheView, CallBinding, FeedForward, Mixer, Norm, Part,
                   PositionEncoding, StateRequest, StepContext)
from .block import PreNormBlock
from .linear import Linear
from .mlp import GatedMlp
from .norm import RmsNorm
from .rotary import NoPosition, Rotary

register_part("norm", "rms_norm", RmsNorm, replace=True)
register_part("position", "rotary", Rotary, replace=True)
register_part("position", "none", NoPosition, replace=True)
register_part("mixer", "attention", Attention, replace=True)
register_part("feed_forward", "gated_mlp", GatedMlp, replace=True)
register_part("block", "pre_norm", lambda layer: PreNormBlock(layer), replace=True)
