"""Parts a model is put together from; importing the package registers the built-in kinds."""
from .base import (Arrangement, FeedForward, LayerCall, LayerSpec, Mixer, ModelPlan, Norm, PagedKvSpec,
                   Part, PartSpec, PositionEncoding, RotaryTable, StateSpec, StepPlan, TensorSource, iter_parts,
                   make_part, register_arrangement, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position, registered)
from . import norm, position, attention, feed_forward, block  # noqa: F401  (registration)
