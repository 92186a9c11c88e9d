"""Sparsity and recall of the operator against dense softmax attention.

The definitions are the reference's: recall at threshold t is the fraction of
output elements whose absolute difference to the dense causal attention output
is below t (anchor_attn/src/ops/ops_profile_v2.py:514-532, thresholds 0.01 and
0.005 in its profiles); the sparsity ratio is the selected query-key pairs over
half of N*N/(block_size*step) per head (anchor_attn/src/ops/anchor_attn_v4.py:271).
``density`` is the share of candidate columns ``[128, b*G-128)`` that step 2
selected.

    python -m anchor_attention_b200.analysis --shape qwen2.5-7b --seq 65536 --thetas 10,12,14
    python -m anchor_attention_b200.analysis --shape llama3.1-8b --seq 32768 --thetas 8,9,10,11,12 --q-shift 0.5
    python -m anchor_attention_b200.analysis --shape llama3.1-8b --seq 32768 --block-thetas 0.05,0.1,0.2 --q-shift 0.5

``--block-thetas`` adds the ablation the reference runs next to it: the block-granular
comparator in its difference-aware mode (``block_sparse.py``; its sparsity ratio is the
listed blocks over the causal blocks, block_sparse_flash_attention_v2.py:301-306) with the same
recall measures.

The dense comparator is torch's scaled_dot_product_attention (a library kernel;
it is only the yardstick).  Inputs are the seeded synthetic tensors of
``synthetic.make_inputs``; ``--q-shift`` selects the auxiliary distribution on
which the selection is actually sparse.
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, Iterable, List

import torch
import torch.nn.functional as F

SHAPES = {"llama3.1-8b": (32, 8), "qwen2.5-7b": (28, 4)}
RECALL_THRESHOLDS = (0.01, 0.005)


def dense_causal(Q, K, V, sm_scale=None) -> torch.Tensor:
    """Dense causal softmax attention of Q [B,H,N,D] over K, V [B,Hkv,N,D]."""
    return F.scaled_dot_product_attention(Q, K, V, is_causal=True, scale=sm_scale, enable_gqa=True)


def recall(out: torch.Tensor, dense: torch.Tensor, threshold: float) -> float:
    return float(((out.float() - dense.float()).abs() < threshold).sum().item() / out.numel())


def candidate_columns(N: int, H: int, block_size: int = 128, step: int = 16, B: int = 1) -> int:
    G = block_size * step
    return B * H * sum(b * G - 2 * block_size for b in range(1, N // G))


def theta_sweep(Q, K, V, thetas: Iterable[float], block_size: int = 128, step: int = 16) -> List[Dict]:
    """One row per theta: density, the reference's sparsity ratio, recall at both
    thresholds, mean/max absolute difference to dense attention, per-head density range."""
    from .ops import AnchorAttnCall
    B, H, N, _ = Q.shape
    dense = dense_causal(Q, K, V)
    cap = candidate_columns(N, H, block_size, step, B)
    G = block_size * step
    cap_head = cap // (B * H)
    rows = []
    for th in thetas:
        call = AnchorAttnCall(Q, K, V, None, block_size, step, th)
        out = call.run()
        call.check_status()
        per_head = call.counts.sum(dim=2).float() / max(cap_head, 1)
        diff = (out.float() - dense.float()).abs()
        row = {"theta": th, "selected_columns": int(call.counts.sum()),
               "density": float(call.counts.sum()) / cap if cap else 0.0,
               "sparsity_ratio": float(call.ratio()),
               "density_per_head_min": float(per_head.min()), "density_per_head_max": float(per_head.max()),
               "density_per_head": [round(float(x), 4) for x in per_head.flatten()],
               "mean_abs_diff": float(diff.mean()), "max_abs_diff": float(diff.max())}
        for t in RECALL_THRESHOLDS:
            row[f"recall@{t}"] = float((diff < t).sum().item() / diff.numel())
        rows.append(row)
        del call, out, diff
    return rows


def block_sparse_sweep(Q, K, V, thetas: Iterable[float], top_k: int = 1 << 30) -> List[Dict]:
    """One row per theta of the block-granular comparator, difference-aware mode: its sparsity
    ratio, recall at both thresholds and mean/max absolute difference to dense attention."""
    from .block_sparse import block_sparse_attention
    dense = dense_causal(Q, K, V)
    rows = []
    for th in thetas:
        out, ratio = block_sparse_attention(Q, K, V, top_k, mode="top_difference_aware", theta=th,
                                            return_sparsity_ratio=True)
        diff = (out.float() - dense.float()).abs()
        row = {"block_theta": th, "top_k": min(top_k, Q.shape[2] // 128), "sparsity_ratio": float(ratio),
               "mean_abs_diff": float(diff.mean()), "max_abs_diff": float(diff.max())}
        for t in RECALL_THRESHOLDS:
            row[f"recall@{t}"] = float((diff < t).sum().item() / diff.numel())
        rows.append(row)
        del out, diff
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="qwen2.5-7b", choices=sorted(SHAPES))
    ap.add_argument("--seq", type=int, default=65536)
    ap.add_argument("--thetas", default="10,12,14")
    ap.add_argument("--block-thetas", default="", help="also sweep the block-granular comparator over these thetas")
    ap.add_argument("--block-top-k", type=int, default=1 << 30)
    ap.add_argument("--q-shift", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the analysis harness needs a CUDA device: the operator has no CPU path")
    from .synthetic import make_inputs
    H, Hkv = SHAPES[args.shape]
    Q, K, V = make_inputs(args.seq, H, Hkv, seed=args.seed, rope=True, q_shift=args.q_shift, device="cuda")
    rows = theta_sweep(Q, K, V, [float(x) for x in args.thetas.split(",")]) if args.thetas else []
    result = {"shape": args.shape, "heads": [H, Hkv], "seq": args.seq, "q_shift": args.q_shift,
              "data": "synthetic", "rows": rows}
    if args.block_thetas:
        result["block_sparse_rows"] = block_sparse_sweep(Q, K, V, [float(x) for x in args.block_thetas.split(",")],
                                                         args.block_top_k)
    print(json.dumps(result))


if __name__ == "__main__":
    main()
