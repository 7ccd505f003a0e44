"""Parts of a decoder and their registries; importing this package registers the built-in kinds."""

from .base import (BLOCKS, DeferredNorm, EMBEDDINGS, FEED_FORWARDS, HEADS, INJECTIONS, Injection, MIXERS, NORMS, POSITION_ENCODINGS, Block,
                   CacheBinding, Embedding, FeedForward, FollowNorm, GroupView, Head, Mixer, Norm, PagedKeyValueNeed, PagedKVNeed, PagedNeed, Part, PreparedNorm,
                   PositionEncoding, Registry, ResidualStream, Runtime, StateNeed, StepContext)
from . import (attention, block, conv_attention, embedding, experts, injection, mlp, norm, normed_attention, recurrent,  # noqa: F401
               rotary)  # noqa: F401  (registration)
from .linear import Linear
