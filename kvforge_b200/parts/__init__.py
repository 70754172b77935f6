"""The parts a model is put together from.  Importing the package registers the built-in
ones (token embedding, rotary encoding, RMSNorm over one or several residual streams, paged
attention, latent attention, the gated delta rule, retention, mixers side by side, gated feed-forward, routed
experts, the pre-norm block over one or several streams, the parallel block, linear head)."""

from . import attention, block, delta, embedding, experts, head, latent, mlp, norm, parallel, retention, rope, talking  # noqa: F401  (registration)
from .base import (  # noqa: F401
    CacheNeed,
    LayerCache,
    PartSpec,
    WeightDecl,
    register_block,
    register_embedding,
    register_feed_forward,
    register_head,
    register_mixer,
    register_norm,
    register_position_encoding,
)
from .model import DecoderModel, LayerCall, LayerSpec, ModelSpec  # noqa: F401
