"""Module hook: swap anchor attention into a Hugging Face model's attention forward.

Mirrors ``patch_model(model, pattern, config)`` of the reference
(anchor_attn/src/modules/patch.py:312-327) for the one pattern this library
implements, with the reference's configuration keys and defaults
(``block_size_M=128, theta=12, step=16``, patch.py:36-45) and its handling of
JSON-string configurations (patch.py:62-74).

The reference binds a new bound-method ``forward`` on every
``LlamaFlashAttention2`` of transformers 4.45
(anchor_attn/src/modules/llama/anchor_attention.py:17-117).  Current
transformers releases route attention through a registry of functions
``fn(module, query[B,H,N,D], key[B,Hkv,N,D], value, attention_mask, scaling,
dropout, **kw) -> (out[B,N,H,D], None)``; this module registers one and points
the model's configuration at it.  The routing rules inside are the reference's
(anchor_attention.py:72-113):

* prefill (q_len > 1, no earlier cache): the first ``q_len - q_len % (step*block)``
  tokens go through ``anchor_attn``; the remaining ``pad`` queries attend densely
  and causally over all keys;
* decode and chunked prefill: dense causal attention.

One intentional divergence: when ``q_len`` is an exact multiple of
``step*block`` the reference slices ``x[:, :-0]``, which is empty, and leaves the
layer's attention output at zero; here ``pad == 0`` means every token goes
through ``anchor_attn``.
"""
from __future__ import annotations

import copy
import json
from typing import Optional

import torch
import torch.nn.functional as F

ATTENTION_CONFIG_EXAMPLE = {
    "anchor_attn": {"block_size_M": 128, "theta": 12, "step": 16},
    "anchor_attn_lite": {"block_size_M": 128, "theta": 12, "step": 16},
}
ATTN_IMPLEMENTATION_NAME = "anchor_attn"
MLP_CHUNK = 32768    # tokens per MLP chunk, as anchor_attn/src/modules/llama/llama_mlp_forward.py:49-56


def get_config_example(pattern: str = None):
    if pattern is None:
        return copy.deepcopy(ATTENTION_CONFIG_EXAMPLE)
    return copy.deepcopy(ATTENTION_CONFIG_EXAMPLE[pattern])


def resolve_config(pattern: str, cfg=None) -> dict:
    """Defaults merged under the caller's dict or JSON string (patch.py:62-74)."""
    if pattern not in ATTENTION_CONFIG_EXAMPLE:
        raise ValueError(f"Unsupported attention pattern {pattern!r}: this library implements "
                         f"{sorted(ATTENTION_CONFIG_EXAMPLE)} only")
    if cfg is None:
        return get_config_example(pattern)
    if isinstance(cfg, str):
        try:
            cfg = json.loads(cfg)
        except json.JSONDecodeError as e:
            raise ValueError(f"Configuration string is not valid JSON: {e}")
    cfg = dict(cfg)
    for k, v in get_config_example(pattern).items():
        cfg.setdefault(k, v)
    return cfg


def patch_model_config(model, pattern: str, cfg=None):
    """Write the hyper-parameters onto ``model.config`` as attributes, where the
    attention function reads them (patch.py:106-109, anchor_attention.py:74,96-98)."""
    cfg = resolve_config(pattern, cfg)
    for k, v in cfg.items():
        setattr(model.config, k, v)
    return cfg


DENSE_CHUNK = 4096   # queries per SDPA call of the dense path: bounds the boolean mask to 4096 x kv_len
DENSE_KERNEL_MIN_Q = 16   # from this many queries on the dense path runs on the library's own kernel


def _dense_causal(query, key, value, scaling, q_offset):
    """Dense causal attention of ``query`` (positions q_offset .. q_offset+q-1) over
    all keys; the path of the tail and of decode (the reference calls flash-attn here,
    anchor_attention.py:76-88,101-113).  Returns [B,H,q,D].
    With DENSE_KERNEL_MIN_Q or more queries (the tail of a prefill, a later prefill chunk) on a
    GPU it runs on the library's own attention kernel (``ops.dense_causal_attention``).  Decode
    (a few queries) and CPU tensors go to torch SDPA, in chunks of DENSE_CHUNK queries so that the
    mask stays small; a query chunk only sees the keys up to its own last position."""
    q_len, kv_len = query.shape[2], key.shape[2]
    if (query.is_cuda and q_len >= DENSE_KERNEL_MIN_Q and query.dtype == torch.bfloat16 and query.shape[3] == 128
            and q_offset + q_len == kv_len):
        from .ops import dense_causal_attention
        return dense_causal_attention(query, key, value, scaling)
    outs = []
    for c0 in range(0, q_len, DENSE_CHUNK):
        c1 = min(q_len, c0 + DENSE_CHUNK)
        hi = min(kv_len, q_offset + c1)                      # keys past the chunk's last query are masked anyway
        pos_q = torch.arange(q_offset + c0, q_offset + c1, device=query.device)[:, None]
        mask = torch.arange(hi, device=query.device)[None, :] <= pos_q
        outs.append(F.scaled_dot_product_attention(query[:, :, c0:c1], key[:, :, :hi], value[:, :, :hi],
                                                   attn_mask=mask, scale=scaling, enable_gqa=True))
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=2)


_head_parallel_group = None
_head_parallel_on = False
_head_parallel_exchange = "push"
_head_parallel_ops = {}


def set_head_parallel_group(group, exchange: str = "push"):
    """Run the sparse part of every patched attention layer head-parallel over the
    ranks of ``group`` (a torch.distributed process group; ``None`` switches it off):
    each rank computes its KV-head groups and the head outputs reach every rank either
    by step 3 storing them into all ranks' output copies ("push") or by one NCCL
    all-gather ("all_gather").  Every rank must call the model with the same inputs."""
    global _head_parallel_group, _head_parallel_on, _head_parallel_exchange
    _head_parallel_group = group
    _head_parallel_on = group is not None
    _head_parallel_exchange = exchange
    _head_parallel_ops.clear()


def _head_parallel_anchor_attn(query, key, value, scaling, block, step, theta, _ratio):
    """anchor_attn on this rank's heads, then the all-gather; returns [B,H,N,D] (a view
    of token-major memory)."""
    import torch.distributed as dist
    from .parallel import HeadShardedAnchorAttn, head_partition
    W, rank = dist.get_world_size(_head_parallel_group), dist.get_rank(_head_parallel_group)
    B, H, N, D = query.shape
    q_lo, q_hi, kv_lo, kv_hi = head_partition(H, key.shape[1], W, rank)
    key_ = (scaling, block, step, theta)
    op = _head_parallel_ops.get(key_)
    if op is None:
        op = _head_parallel_ops[key_] = HeadShardedAnchorAttn(scaling, block, step, theta, _head_parallel_group,
                                                              exchange=_head_parallel_exchange)
    return op(query[:, q_lo:q_hi], key[:, kv_lo:kv_hi], value[:, kv_lo:kv_hi]).permute(0, 2, 1, 3)


def anchor_attention_forward(module, query, key, value, attention_mask=None, scaling: Optional[float] = None,
                             dropout: float = 0.0, anchor_attn_fn=None, **kwargs):
    """Attention function for the transformers attention registry.
    query [B,H,N,D]; key, value [B,Hkv,Nk,D]; returns ([B,N,H,D], None)."""
    if anchor_attn_fn is None and _head_parallel_on:
        anchor_attn_fn = _head_parallel_anchor_attn
    cfg = module.config
    block, step, theta = int(cfg.block_size_M), int(cfg.step), float(cfg.theta)
    B, H, q_len, D = query.shape
    kv_len = key.shape[2]
    G = block * step
    out = torch.empty((B, q_len, H, D), dtype=query.dtype, device=query.device)
    n_sparse = (q_len - q_len % G) if (q_len > 1 and q_len == kv_len) else 0
    if n_sparse and anchor_attn_fn is None:
        # the kernels read the [B,N,H,D]-ordered projections through their strides and write
        # the token-major result in place: no transposes, no repeat_kv
        from .ops import AnchorAttnCall
        AnchorAttnCall(query[:, :, :n_sparse], key[:, :, :n_sparse], value[:, :, :n_sparse], scaling, block, step,
                       theta, out=out[:, :n_sparse].permute(0, 2, 1, 3)).run()
    elif n_sparse:
        sparse = anchor_attn_fn(query[:, :, :n_sparse], key[:, :, :n_sparse], value[:, :, :n_sparse],
                                scaling, block, step, theta, False)
        out[:, :n_sparse] = sparse.transpose(1, 2)
    if n_sparse < q_len:
        tail = _dense_causal(query[:, :, n_sparse:], key, value, scaling, kv_len - (q_len - n_sparse))
        out[:, n_sparse:] = tail.transpose(1, 2)
    return out, None


def _chunked_mlp_forward(mlp):
    inner = mlp.forward

    def forward(x):
        if x.dim() != 3 or x.shape[1] <= MLP_CHUNK:
            return inner(x)
        return torch.cat([inner(x[:, i:i + MLP_CHUNK]) for i in range(0, x.shape[1], MLP_CHUNK)], dim=1)

    return forward


def patch_model(model, pattern: str, config=None):
    """Patch a Hugging Face causal LM to use anchor attention for prefill.
    ``pattern`` must be "anchor_attn" (or its alias "anchor_attn_lite", which the
    reference maps to the same forward, patch.py:142-144)."""
    from transformers import AttentionInterface, PreTrainedModel
    if not isinstance(model, PreTrainedModel):
        raise ValueError("Only Hugging Face transformers models are supported")
    name = type(model).__name__.lower()
    if not any(t in name for t in ("llama", "qwen2", "qwen3", "mistral")):
        raise ValueError(f"Unsupported model type: {type(model).__name__}")
    # the dense path (tail, decode) is plain causal attention: a model that restricts attention
    # to a sliding window would silently get full attention there (the reference hands
    # sliding_window to its dense call, modules/llama/anchor_attention.py:76-88)
    window = getattr(model.config, "sliding_window", None)
    if window is not None and getattr(model.config, "use_sliding_window", True):
        raise ValueError(f"models with a sliding attention window (sliding_window={window}) are not supported")
    patch_model_config(model, pattern, config)
    AttentionInterface.register(ATTN_IMPLEMENTATION_NAME, anchor_attention_forward)
    model.config._attn_implementation = ATTN_IMPLEMENTATION_NAME
    install_chunked_mlp(model)
    return model


def install_chunked_mlp(model):
    """The memory patch the reference applies with every pattern: each MLP runs in
    32768-token chunks (anchor_attn/src/modules/llama/llama_mlp_forward.py:49-56)."""
    for mod in model.modules():
        if type(mod).__name__.endswith("MLP") and not getattr(mod, "_anchor_chunked", False):
            mod.forward = _chunked_mlp_forward(mod)
            mod._anchor_chunked = True
    return model
