"""B200-native anchor attention: the reference's ``anchor_attn`` prefill operator
backed by hand-written sm_100a CUDA kernels behind a C ABI."""
from .ops import (AnchorAttnCall, anchor_attn, anchor_attn_host, anchor_attn_test_time,
                  anchor_attn_without_anchor, dense_causal_attention, launches_per_forward)


def __getattr__(name):
    # the block-granular comparator is imported on first use
    if name == "block_sparse_attention":
        from .block_sparse import block_sparse_attention
        return block_sparse_attention
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

__all__ = ["anchor_attn", "anchor_attn_without_anchor", "anchor_attn_test_time", "anchor_attn_host",
           "AnchorAttnCall", "dense_causal_attention", "launches_per_forward", "block_sparse_attention"]
