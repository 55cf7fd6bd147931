"""Parts a decoder is assembled from.  Importing this package registers the built-in kinds."""
from . import (attention, block, latent_attention, min_gru, mlp, moe, norm, retention, rope, selective_scan,  # noqa: F401
               side_by_side)
from .base import (Block, CacheView, FeedForward, HostBatch, Mixer, Norm, Part, PositionEncoding, StepContext,
                   WeightSpec)
