"""Parts of a model (norm, position encoding, mixer, feed-forward, block, embedding, head)
and the model that a plan puts together from them."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, STREAMS, Part, build_part,
                   register_part)
from . import (norm, position, attention, differential, lightning, latent, gated_recurrence, gated_linear, matrix_memory, parallel, mlp, moe,  # noqa: F401
               block, embedding, stream)  # noqa: F401  (registration)
from .model import Model, build_model

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "STREAMS", "Part", "build_part",
           "register_part", "Model", "build_model"]
