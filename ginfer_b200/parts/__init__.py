"""Parts a model is put together from: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (Block, Embedding, FeedForward, Head, LazyNorm, Mixer, Norm, PagedKVBinding,
                   PagedKVSpec, Part, PositionEncoding, StateBinding, StateSpec, StepContext, Summed,
                   TensorSpec,
                   make_part, register_block, register_feed_forward, register_mixer,
                   register_norm, register_part, register_position)
from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry, sequential_run
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register)
from .model import DecoderModel
