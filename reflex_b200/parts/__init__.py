from .registry import (  # noqa: F401
    BLOCKS,
    EMBEDDING_TERMS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITIONS,
    Rotation,
    TensorInfo,
    register_block,
    register_embedding_term,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position,
)
from . import norm, rope, mlp, attention, block, embedding, latent_attention, mlstm, moe  # noqa: F401,E402
from . import conv_attention, rglru, pair  # noqa: F401,E402  (registers the parts)
from . import hyper, selective_scan  # noqa: F401,E402
from . import sigmoid_attention, ssd, delta_rule  # noqa: F401,E402
