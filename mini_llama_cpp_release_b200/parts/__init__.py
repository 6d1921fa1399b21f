"""The parts models are assembled from.  Importing this package registers the built-in
kinds: norm/rmsnorm, norm/layernorm, position/rope_neox, position/rope_partial, position/none,
mixer/gqa_attention, mixer/sink_attention, mixer/latent_attention, mixer/gated_delta,
mixer/gated_linear_attention, mixer/gated_linear_recurrence, mixer/parallel, feed_forward/swiglu,
feed_forward/mixture, block/prenorm, block/branch_norm, block/parallel, block/stream_mix,
embedding/token_embedding, head/linear_head."""
from .base import CacheNeed, MixerMemory, Part, Runtime, StateSpec, TensorSpec  # noqa: F401
from .linear import Linear  # noqa: F401
from . import norm, rotary, attention, recurrent, feed_forward, block, embedding  # noqa: F401
