"""Parts of a model.  Importing the package registers the built-in kinds."""
from . import attention, feed_forward, latent_attention, model, norm, position, routed_experts  # noqa: F401
