"""Parts a decoder is composed of, their specifications and registries."""
from . import specs
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Part, Registry, Runtime
from . import norm, position, attention, latent_attention, linear_attention, matrix_memory, time_mix, state_space, delta_rule, mixer_pair, feedforward, block, embedding  # register the built-in kinds

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Part", "Registry", "Runtime", "specs"]
