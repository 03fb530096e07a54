"""CPU oracle for the ReDrafter decode step.  TEST INFRASTRUCTURE ONLY.

This package restates, in plain numpy (fp32 / int64), the algorithm of the
speculative-decoding step of apple/ml-recurrent-drafter:

    drafter beam search -> prefix-tree dedup/pack/mask -> Llama verify forward
    -> acceptance (greedy / speculative sampling) -> KV-cache + input_ids commit.

Every function cites the reference file:line it follows.  The restatement is
pinned against (a) the golden tensors held by the reference's own unit tests
and (b) outputs of the reference's PyTorch code run on CPU on seeded inputs;
both sets are committed under tests/golden/ together with the script that
produced them (tests/golden/make_golden.py).

Nothing in the product package may import this package.  It is used by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the
checker / the timed CPU baseline, never as the thing shipped.
"""

from . import acceptance, drafter, generate, kv_cache, llama, tree_attention  # noqa: F401
