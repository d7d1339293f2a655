"""Parts of a layer. Importing this package registers the built-in parts."""
from . import (base, rmsnorm, layernorm, rotary, attention, latent_attention, recurrent, decayed_attention, delta_rule, constant_decay, shifted_mixing, side_by_side, swiglu, dense_ff,
               routed_ff, gate, block, vocab)  # noqa: F401
from .base import (Block, CompositeNeed, DeferredNorm, Embedding, FeedForward, Gate, Head, Mixer, Norm, PagedKVNeed, Part,
                   PositionEncoding, StateNeed, register_gate, build_part, part_class, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position, unregister)
