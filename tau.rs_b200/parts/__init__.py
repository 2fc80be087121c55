from . import (attention, block, delta_rule, differential_attention, latent_attention, linear_recurrence, masked_attention, mlp, norm, rope,
               routed_experts, selective_scan, side_by_side, wkv)  # noqa: F401  (registers the kinds)
from .base import Block, CacheNeed, FeedForward, Mixer, Norm, Part
from .linear import StackedLinear
from .model import DecoderModel
from .registry import (build, register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, unregister)
