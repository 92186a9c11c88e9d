"""The block-granular comparator of the reference, backed by the CUDA library.

The reference measures anchor attention against block-sparse flash attention in
which every 128-row query block attends a list of whole 128-row key blocks
(anchor_attn/src/ops/block_sparse_flash_attention_v2.py).  This module mirrors it:

* ``block_sparse_attention`` -- the wrapper (:311-356): same name, signature, defaults,
  modes (``top_k``, ``top_cdf``, ``top_difference_aware``) and return convention;
* ``build_block_index*`` -- the three index builders (:150-309).  Like the reference's they
  are a few tensor operations on the block-mean queries and keys (a [N/128, N/128] score
  matrix per head); the per-row Python loops that pack the lists are replaced by one
  scatter, the produced ``block_index`` is the same tensor;
* ``block_sparse_attend`` -- the attention itself (:113-144, kernel :10-110) through the C
  ABI (``aa_block_sparse_attend``), on any ``block_index`` in the reference's format.

K and V may carry fewer heads than Q (grouped-query attention).  Block sizes other than
128 x 128 are not supported (no harness of the reference uses another).

    python -m anchor_attention_b200.block_sparse --seq 32768 --mode top_k --top-k 64

times the builder and the attention on seeded synthetic tensors (CUDA events) and prints one
JSON line.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .ops import _usable, _workspace

__all__ = ["block_sparse_attention", "block_sparse_attend", "build_block_index",
           "build_block_index_top_cdf", "build_block_index_difference_aware"]

BLOCK = 128


# --------------------------------------------------------------------------- index builders
def _pooled_scores(query, key, scale: Optional[float]):
    """Block-mean queries (times ``scale`` if given) against block-mean keys, blocks above the
    diagonal set to -inf: [B, H, N/128, N/128] in the input dtype
    (block_sparse_flash_attention_v2.py:166-174, 211-217, 267-273)."""
    B, H, N, D = query.shape
    Hkv = key.shape[1]
    nb = N // BLOCK
    qp = query.reshape(B, H, nb, BLOCK, D).mean(dim=-2)
    if scale is not None:
        qp = qp * scale
    kp = key.reshape(B, Hkv, nb, BLOCK, D).mean(dim=-2)
    if Hkv != H:
        kp = kp.repeat_interleave(H // Hkv, dim=1)
    p = torch.einsum('bhmk,bhnk->bhmn', qp, kp)
    start = torch.arange(nb, device=query.device) * BLOCK
    return p.masked_fill(start[None, None, :, None] < start[None, None, None, :], float('-inf'))


def _pack(valid: torch.Tensor, max_blocks: int) -> torch.Tensor:
    """Rows of ``valid`` [B,H,nb,nb] as ascending index lists of width ``max_blocks``: a row
    with c selected blocks becomes max_blocks - c zeros followed by its c indices, which is what
    zero-initialising, filling the first c slots and sorting gives
    (block_sparse_flash_attention_v2.py:228-239, 294-305)."""
    counts = valid.sum(dim=-1, dtype=torch.int32)
    out = torch.zeros(valid.shape[:-1] + (max_blocks,), dtype=torch.int32, device=valid.device)
    rank = valid.cumsum(dim=-1, dtype=torch.int32) - 1
    b, h, m, n = torch.nonzero(valid, as_tuple=True)
    pos = (max_blocks - counts[b, h, m] + rank[b, h, m, n]).long()
    out[b, h, m, pos] = n.int()
    return out


def _ratio(total_used: int, B: int, H: int, nb: int) -> float:
    total_possible = B * H * nb * (nb + 1) // 2
    return total_used / total_possible if total_possible > 0 else 0.0


def build_block_index(query, key, top_k: int, block_size_M: int = BLOCK, block_size_N: int = BLOCK):
    """The ``top_k`` mode: the k best key blocks of every query block by block-mean score
    (block_sparse_flash_attention_v2.py:150-190).  Returns ``(block_index int32
    [B,H,nb,k], sparsity_ratio)``."""
    assert block_size_M == BLOCK and block_size_N == BLOCK, "only 128 x 128 blocks are supported"
    B, H, N, _ = query.shape
    nb = N // BLOCK
    p = _pooled_scores(query, key, None)
    top_k = nb if top_k >= nb else int(top_k)
    block_index = torch.topk(p, top_k, dim=-1).indices.sort(dim=-1).values
    total_used = B * H * ((nb - top_k) * top_k + top_k * (top_k + 1) // 2)
    return block_index.int(), _ratio(total_used, B, H, nb)


def build_block_index_top_cdf(query, key, cdf_threshold: float = 0.95, block_size_M: int = BLOCK,
                              block_size_N: int = BLOCK, sm_scale: float = None):
    """The ``top_cdf`` mode: the leading key blocks of every row up to where the cumulative
    softmax of the block-mean scores passes the threshold
    (block_sparse_flash_attention_v2.py:193-243)."""
    assert block_size_M == BLOCK and block_size_N == BLOCK, "only 128 x 128 blocks are supported"
    B, H, N, _ = query.shape
    nb = N // BLOCK
    p = _pooled_scores(query, key, sm_scale)
    cdf = torch.softmax(p, dim=-1).cumsum(dim=-1)
    cutoff = (cdf > cdf_threshold).float().argmax(dim=-1) + 1
    n_idx = torch.arange(nb, device=query.device)
    valid = (n_idx[None, None, None, :] < cutoff[..., None]) & (n_idx[None, None, :, None] >= n_idx[None, None, None, :])
    counts = valid.sum(dim=-1)
    block_index = _pack(valid, int(counts.max().item()))
    return block_index, _ratio(int(counts.sum().item()), B, H, nb)


def build_block_index_difference_aware(query, key, block_size_M: int = BLOCK, block_size_N: int = BLOCK,
                                       theta: float = 0.5, sm_scale: float = None, top_k: int = 1 << 30):
    """The ``top_difference_aware`` mode: the key blocks whose block-mean score lies within
    ``theta`` of the row's best one, the best one always included, at most ``top_k`` of them
    (block_sparse_flash_attention_v2.py:246-309).  ``top_k`` must be finite (the reference's
    default, infinity, fails at its ``int(top_k)``, :294)."""
    assert block_size_M == BLOCK and block_size_N == BLOCK, "only 128 x 128 blocks are supported"
    B, H, N, _ = query.shape
    nb = N // BLOCK
    top_k = int(min(top_k, 1 << 30))
    p = _pooled_scores(query, key, sm_scale)
    best = p.max(dim=-1, keepdim=True).values
    valid = (best - p) <= theta
    valid.scatter_(-1, p.argmax(dim=-1, keepdim=True), True)
    if top_k < nb:
        scores = p.masked_fill(~valid, float('-inf'))
        keep = scores.topk(min(top_k, nb), dim=-1).indices
        valid = torch.zeros_like(valid).scatter_(-1, keep, True)
    counts = valid.sum(dim=-1)
    max_blocks = min(int(counts.max().item()), top_k)
    block_index = _pack(valid, max_blocks)
    return block_index, _ratio(int(counts.sum().item()), B, H, nb)


# --------------------------------------------------------------------------- the attention
def block_sparse_attend(q, k, v, block_index, sm_scale: float = None, out: Optional[torch.Tensor] = None,
                        check: bool = False):
    """Block-sparse flash attention on a given ``block_index`` (int32 [B,H,N/128,max_blocks],
    rows ascending): the reference's ``_triton_block_sparse_attention``
    (block_sparse_flash_attention_v2.py:113-144) with every row of q valid.  q [B,H,N,128];
    k, v [B,H or Hkv,N,128]; bf16 CUDA tensors, N a multiple of 256.  Returns the [B,H,N,128]
    output; the launches are asynchronous on the current stream unless ``check`` is set, which
    synchronises and raises if a list was not ascending or a device-side wait gave up."""
    lib = _lib.load()
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be [B, H, N, D]"
    assert q.is_cuda and k.is_cuda and v.is_cuda, "q, k, v must be CUDA tensors (there is no CPU path)"
    assert q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype, "q, k, v must be bfloat16"
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    assert D == 128, f"head dimension {D} is not supported (128 only)"
    assert k.shape == v.shape and k.shape[0] == B and k.shape[2] == N and k.shape[3] == D, \
        "k and v must be [B, Hkv, N, D] with the batch, length and head size of q"
    assert H % Hkv == 0, f"{Hkv} KV heads do not divide {H} query heads"
    assert N % (2 * BLOCK) == 0, f"sequence length {N} must be a multiple of {2 * BLOCK}"
    assert block_index.dim() == 4 and tuple(block_index.shape[:3]) == (B, H, N // BLOCK) and block_index.shape[3] >= 1, \
        f"block_index must be [B, H, N/{BLOCK}, max_blocks]"
    assert block_index.is_cuda and block_index.device == q.device, "block_index must live on q's device"
    bi = block_index.to(torch.int32).contiguous()
    q, k, v = _usable(q), _usable(k), _usable(v)
    if out is None:
        out = torch.empty((B, H, N, D), dtype=q.dtype, device=q.device)
    a = _lib.AABlockSparse()
    a.B, a.H, a.Hkv, a.N, a.D = B, H, Hkv, N, D
    a.dtype, a.max_blocks = _lib.AA_BF16, bi.shape[3]
    a.sm_scale = float(sm_scale) if sm_scale else 0.0
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    for name, t in (("q", q), ("k", k), ("v", v), ("o", out)):
        setattr(a, f"{name}_stride_b", t.stride(0))
        setattr(a, f"{name}_stride_h", t.stride(1))
        setattr(a, f"{name}_stride_n", t.stride(2))
    a.block_index = bi.data_ptr()
    need = ctypes.c_size_t(0)
    rc = lib.aa_block_sparse_workspace_bytes(ctypes.byref(a), ctypes.byref(need))
    if rc != _lib.AA_OK:
        raise AssertionError(_lib.error_text(rc))
    stream = torch.cuda.current_stream(q.device)
    ws = _workspace(q.device, stream.cuda_stream, need.value)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(q.device):
        rc = lib.aa_block_sparse_attend(ctypes.byref(a), ctypes.c_void_p(stream.cuda_stream))
        if rc == _lib.AA_OK and check:
            rc = lib.aa_block_sparse_check_status(ctypes.byref(a), ctypes.c_void_p(stream.cuda_stream))
    if rc != _lib.AA_OK:
        raise RuntimeError(f"block_sparse_attend: {_lib.error_text(rc)}")
    return out


def block_sparse_attention(query, key, value, top_k: int, block_size_M: int = BLOCK, block_size_N: int = BLOCK,
                           mode: str = 'top_k', cdf_threshold: float = 0.95, theta: float = 0.5,
                           return_sparsity_ratio: bool = False):
    """Block-sparse self-attention with one of the three selection modes, as the reference's
    ``block_sparse_attention`` (block_sparse_flash_attention_v2.py:311-356): the inputs are
    zero-padded to whole blocks, the block lists are built from the padded tensors, the
    output is cut back to the input length.  Returns ``out`` or ``(out, sparsity_ratio)``."""
    B, H, L, D = query.shape
    sm_scale = D ** -0.5
    pad = (-L) % block_size_M
    if pad > 0:
        query = torch.nn.functional.pad(query, (0, 0, 0, pad))
        key = torch.nn.functional.pad(key, (0, 0, 0, pad))
        value = torch.nn.functional.pad(value, (0, 0, 0, pad))
    if mode == 'top_k':
        idx, ratio = build_block_index(query, key, top_k, block_size_M, block_size_N)
    elif mode == 'top_cdf':
        idx, ratio = build_block_index_top_cdf(query, key, cdf_threshold, block_size_M, block_size_N, sm_scale)
    elif mode == 'top_difference_aware':
        idx, ratio = build_block_index_difference_aware(query, key, block_size_M, block_size_N, theta, sm_scale, top_k)
    else:
        raise ValueError(f"Unsupported mode: {mode}. Choose 'top_k', 'top_cdf', or 'top_difference_aware'.")
    if (query.shape[2] // BLOCK) % 2:
        # the kernel works on pairs of query blocks: one more block of zero rows whose list is
        # key block 0 and whose output is cut off again
        query = torch.nn.functional.pad(query, (0, 0, 0, BLOCK))
        key = torch.nn.functional.pad(key, (0, 0, 0, BLOCK))
        value = torch.nn.functional.pad(value, (0, 0, 0, BLOCK))
        idx = torch.nn.functional.pad(idx, (0, 0, 0, 1))
    out = block_sparse_attend(query, key, value, idx, sm_scale)[..., :L, :]
    return (out, ratio) if return_sparsity_ratio else out


def main():
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--heads", default="32,8")
    ap.add_argument("--mode", default="top_k", choices=["top_k", "top_cdf", "top_difference_aware", "dense"])
    ap.add_argument("--top-k", type=int, default=64)
    ap.add_argument("--theta", type=float, default=0.5)
    ap.add_argument("--cdf-threshold", type=float, default=0.95)
    ap.add_argument("--q-shift", type=float, default=0.0)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the attention has no CPU path")
    from .synthetic import make_inputs
    H, Hkv = (int(x) for x in args.heads.split(","))
    N = args.seq
    Q, K, V = make_inputs(N, H, Hkv, seed=0, rope=True, q_shift=args.q_shift, device="cuda")
    nb = N // BLOCK
    sm = Q.shape[-1] ** -0.5
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    if args.mode == "dense":
        idx = torch.arange(nb, dtype=torch.int32, device="cuda").expand(1, H, nb, nb).contiguous()
        ratio = 1.0
    elif args.mode == "top_k":
        idx, ratio = build_block_index(Q, K, args.top_k)
    elif args.mode == "top_cdf":
        idx, ratio = build_block_index_top_cdf(Q, K, args.cdf_threshold, BLOCK, BLOCK, sm)
    else:
        idx, ratio = build_block_index_difference_aware(Q, K, BLOCK, BLOCK, args.theta, sm, args.top_k)
    ev[1].record()
    for _ in range(args.warmup):
        block_sparse_attend(Q, K, V, idx, sm)
    ev[2].record()
    for _ in range(args.steps):
        out = block_sparse_attend(Q, K, V, idx, sm)
    ev[3].record()
    block_sparse_attend(Q, K, V, idx, sm, out=out, check=True)
    ms = ev[2].elapsed_time(ev[3]) / args.steps
    # entries the kernel reads: min(m + 1, max_blocks) per query block (block_sparse_flash_attention_v2.py:66)
    read = int(torch.minimum(torch.arange(1, nb + 1), torch.tensor(idx.shape[-1])).sum()) * H
    print(json.dumps({"workload": f"block-sparse attention, seq {N}, {H}q/{Hkv}kv heads, mode {args.mode}",
                      "max_blocks": int(idx.shape[-1]), "sparsity_ratio": float(ratio),
                      "builder_ms": ev[0].elapsed_time(ev[1]), "attend_ms": ms, "entries_read": read,
                      "tflops_on_entries_read": read * 4 * BLOCK ** 3 / ms / 1e9, "steps": args.steps,
                      "data": "synthetic"}))


if __name__ == "__main__":
    main()
