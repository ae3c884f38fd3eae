"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, attention_bias, attention_keys, attention_masked, block, hyper, embedding, latent_attention, mlp, moe, norm, recurrent, rotary, sandwich, wide  # noqa: F401
from .base import register_part, unregister_part  # noqa: F401
