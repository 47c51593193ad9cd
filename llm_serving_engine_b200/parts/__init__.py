from . import (attention, block, branches, latent_attention, linear_attention, mlp, mlstm, moe, norm,  # noqa: F401
               normed_attention, rope)   # (register the built-in parts)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildContext,
                   FeedForward, Mixer, Norm, PagedKV, PagedLatent, Part, PositionEncoding, RequestState,
                   ResidualStream, register_block, register_feed_forward, register_mixer,
                   register_norm, register_position_encoding)
from .linear import linear, linear_partials, reduce_partials

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "BuildContext",
    "FeedForward", "Mixer", "Norm", "PagedKV", "PagedLatent", "Part", "PositionEncoding", "RequestState",
    "ResidualStream", "linear", "linear_partials", "reduce_partials", "register_block", "register_feed_forward", "register_mixer",
    "register_norm", "register_position_encoding",
]
