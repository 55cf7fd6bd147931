"""Parts a decoder is assembled from.  Importing this package registers the built-in kinds."""
from . import attention, block, latent_attention, min_gru, mlp, moe, norm, rope, selective_scan  # noqa: F401
from .base import (Block, CacheView, FeedForward, HostBatch, Mixer, Norm, Part, PositionEncoding, StepContext,
                   WeightSpec)
