"""Parts of a layer.  Importing this package registers the built-in parts."""
from . import attention, block, branches, embedding, ffn, latent_attention, mlstm, norm, recurrent, rope  # noqa: F401
from .base import BuildContext, EmbedAddition, FeedForward, Mixer, Norm, Part, PositionEncoding  # noqa: F401
