"""Helpers shared by the GPU parity tests."""
import torch

from oracle.anchor_oracle import LOG2E, f32, pool_anchor, pool_q

# north-star output tolerance against the reference semantics (bf16)
OUT_MAX_ABS = 2e-2
OUT_MEAN_ABS = 1e-3


def bf16_step(x: torch.Tensor) -> torch.Tensor:
    """Distance between neighbouring bf16 values at the magnitude of each element of x
    (8 significant bits: 2^(floor(log2 |x|) - 7)); zero maps to the smallest step used."""
    e = torch.floor(torch.log2(x.abs().clamp_min(2.0 ** -120)))
    return torch.exp2(e - 7)


def tie_band(q, k, M, sm_scale, theta, b, block_size=128, step=16):
    """Classify the candidate columns of big block b of one head.
    Returns (sure_in, sure_out, band) as boolean masks over columns
    [block_size, b*G - block_size).  A column is in the band when the decision
    score + theta*log2e >= anchor of some pooled row lies within the bf16 rounding
    of the score and of the anchor plus fp32 accumulation-order noise, so two
    correct implementations may disagree on it."""
    G = block_size * step
    qp = pool_q(q, block_size, "bf16", "tree")
    ap = pool_anchor(M, block_size, "bf16", "tree")
    lo, hi = block_size, b * G - block_size
    raw = (qp[b * step:(b + 1) * step] @ k[lo:hi].float().T) * f32(sm_scale * LOG2E)
    a = ap[b * step:(b + 1) * step, None]
    margin = raw + f32(theta * LOG2E) - a
    tol = torch.maximum(raw.abs(), a.abs()) * 2.0 ** -8 + 4e-3
    sure_in = (margin > tol).any(dim=0)
    sure_out = (margin < -tol).all(dim=0)
    return sure_in, sure_out, ~(sure_in | sure_out)


def check_id_set(ours, q, k, M, sm_scale, theta, b, block_size=128, step=16):
    """R \\ T subset of S subset of R U T, with R decided by the exact margins.
    Returns (size of the band, number of band columns we selected)."""
    G = block_size * step
    sure_in, sure_out, band = tie_band(q, k, M, sm_scale, theta, b, block_size, step)
    sel = torch.zeros(b * G - 2 * block_size, dtype=torch.bool)
    sel[ours.long() - block_size] = True
    missing = (sure_in & ~sel).sum().item()
    extra = (sure_out & sel).sum().item()
    assert missing == 0, f"big block {b}: {missing} columns that must be selected are missing"
    assert extra == 0, f"big block {b}: {extra} columns selected that must not be"
    return int(band.sum()), int((band & sel).sum())
