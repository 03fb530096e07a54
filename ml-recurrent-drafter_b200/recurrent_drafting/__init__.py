"""B200-native implementation of the ReDrafter speculative-decoding step behind the Python API of
apple/ml-recurrent-drafter (module names, classes and signatures follow recurrent_drafting/ of the
reference).  Every operator on the decode path runs in hand-written sm_100a CUDA kernels reached
through the C ABI of libredrafter_b200.so; there is no CPU path."""

from . import (  # noqa: F401
    attention,
    autoregressive,
    configuration_drafter,
    kv_cache,
    modeling_drafter,
    modeling_llama,
    recurrent_drafting,
    replicas,
    rng,
    stats,
    tree_attention,
)
from .recurrent_drafting import RecurrentDrafting, SamplingArgs, SpecialTokens  # noqa: F401
