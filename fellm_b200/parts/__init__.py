from . import (attention, connector, dyt, embedding, gated_delta, moe, parallel, retention, rmsnorm, rope,  # noqa: F401
               shortconv, swiglu, timemix)                                                                        # (registers the parts)
from .base import (CONNECTORS, Connector, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Embedding,
                   FeedForward, FixedState, Head, Mixer, Norm, PagedKV, ParamDecl, Part, PositionEncoding,
                   build_part, register_part)
from .spec import LayerSpec, ModelSpec, PartSpec, Run
