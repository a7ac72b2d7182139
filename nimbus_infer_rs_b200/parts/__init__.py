from .base import (INDEX, MATRIX, TABLE, VECTOR, Block, DeferredNorm, FeedForward, KVRequest, Mixer, Norm,
                   ParamSpec, Part, PartSpec, Position, StateRequest, bind_params, build_part,
                   collect_param_specs, register_part, registered_parts)
from .linear import Linear
from .norm import LayerNorm
from .position import LearnedAbsolute, NoPosition
from .embedding import LMHead, TokenEmbedding
from .attention import CausalSelfAttention
from .feed_forward import DenseMLP
from .block import PreNormBlock
