"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""

from . import (attention, bigram, block, channel_delta, differential_attention, feed_forward, latent_attention,  # noqa: F401
               linear_recurrence, norms, pass_entry, rope, routed_experts, side_by_side, time_mix, token_side)
from .base import (BLOCKS, FEED_FORWARDS, LAYER_EXTRAS, MIXERS, NORMS, PASS_ENTRIES, POSITION_ENCODINGS, Block, BuildContext,  # noqa: F401
                   CacheNeeds, FeedForward, KVNeeds, LayerExtra, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, Stage, StateNeeds, TensorSpec)
