"""Parts a model is put together from: mixers, feed-forwards, norms, position
encodings and block arrangements, each registered under a kind and built from a
``PartSpec`` of sizes and constants."""

from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                       BuildContext, register_block, register_embedding, register_feed_forward,
                       register_head, register_mixer, register_norm, register_position_encoding)
from .spec import (LayerSpec, ModelPlan, PagedKVSpec, PartSpec, ScheduleEntry, StateSpec,
                   TensorSpec)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the kinds)
