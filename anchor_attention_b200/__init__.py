"""B200-native anchor attention: the reference's ``anchor_attn`` prefill operator
backed by hand-written sm_100a CUDA kernels behind a C ABI."""
from .ops import (AnchorAttnCall, anchor_attn, anchor_attn_host, anchor_attn_without_anchor,
                  launches_per_forward)

__all__ = ["anchor_attn", "anchor_attn_without_anchor", "anchor_attn_host", "AnchorAttnCall",
           "launches_per_forward"]
