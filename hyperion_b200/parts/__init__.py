from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Arrangement, BuildContext,
                   Embedding, FeedForward, Head, Mixer, Norm, PagedKV, PagedTokens, Part, PositionEncoding, RequestState, WeightSpec,
                   register_arrangement, register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position)
from .spec import LayerSpec, ModelSpec, PartSpec, Run
