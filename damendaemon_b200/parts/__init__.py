from .interfaces import Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Runtime
from .model import DecoderModel, cache_needs, tensor_decls
from .registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, register_arrangement,
                       register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                       register_position)
from .spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, NormSpec,
                   PositionSpec, RunEntry, TensorDecl)
