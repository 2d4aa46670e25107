"""Parts a model is put together from: mixers, feed-forwards, norms, position
encodings and block arrangements, each registered under a kind and built from a
``PartSpec`` of sizes and constants."""

from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, BuildContext,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position_encoding)
from .spec import (LayerSpec, ModelPlan, PagedKVSpec, PartSpec, ScheduleEntry, StateSpec,
                   TensorSpec)
from . import attention, block, feed_forward, norm, position  # noqa: F401  (register the kinds)
