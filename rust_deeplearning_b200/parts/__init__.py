"""Parts of a model.  Importing the package registers the built-in kinds."""
from . import (attention, decay_attention, feed_forward, latent_attention, mixer_pair, model, norm, position,  # noqa: F401
               routed_experts)
