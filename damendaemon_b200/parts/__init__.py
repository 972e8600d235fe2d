from .interfaces import FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime
from .model import DecoderModel, cache_needs, tensor_decls
from .registry import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, register_arrangement,
                       register_feed_forward, register_mixer, register_norm, register_position)
from .spec import (AttentionSpec, DenseFeedForwardSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, RunEntry,
                   TensorDecl)
