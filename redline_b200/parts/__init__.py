"""Parts a layer is put together from.  Importing the package registers the
built-in parts."""

from . import (attention, attention_maps, block, delta_rule, embedding, latent_attention, layernorm,  # noqa: F401
               linear_attention, matrix_memory, mlp, moe, parallel, rmsnorm, rope, streams)
from .base import (Block, Embedding, FeedForward, Head, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   Runtime, Workspace, build_part, lookup, register)
from .spec import CacheSpec, CacheTensor, LayerCall, LayerSpec, ModelSpec, PartSpec, StateSpec, TensorSpec
