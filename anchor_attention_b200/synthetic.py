"""Seeded synthetic Q/K/V with the shapes and value distribution the benchmark
configurations name: N(0,1) entries from a CPU generator, the first 64 key rows
scaled by 4 (attention sink), a random 1 % of key positions shifted by
3*mean(Q) (vertical stripes), HF rotate-half RoPE at base 500000, bf16.
These stand in for the real-model activations the reference profiles from
dumps (anchor_attn/src/ops/ops_profile_v2.py:722-765), which are not available."""
import torch


def rope_rotate_half(x: torch.Tensor, base: float = 500000.0) -> torch.Tensor:
    N, D = x.shape[-2:]
    inv = base ** (-torch.arange(0, D, 2, dtype=torch.float32, device=x.device) / D)
    ang = torch.arange(N, dtype=torch.float32, device=x.device)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    cos, sin = emb.cos(), emb.sin()
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return x * cos + torch.cat([-x2, x1], dim=-1) * sin


def make_inputs(N, H, Hkv, D=128, seed=0, rope=True, dtype=torch.bfloat16, q_shift=0.0, device=None,
                heads=None):
    """Returns (Q [1,H,N,D], K [1,Hkv,N,D], V [1,Hkv,N,D]).  Random numbers are
    always drawn on the CPU (same stream of values everywhere); RoPE and the cast
    run on ``device`` when given.  ``heads=(q_lo, q_hi, kv_lo, kv_hi)`` keeps only
    that slice of heads (every rank of a head-sharded run draws the full tensors
    from the same seed and keeps its own heads)."""
    g = torch.Generator("cpu").manual_seed(seed)
    Q = torch.randn(1, H, N, D, generator=g)
    K = torch.randn(1, Hkv, N, D, generator=g)
    V = torch.randn(1, Hkv, N, D, generator=g)
    if q_shift:
        Q = Q + q_shift
    K[:, :, :64] *= 4
    idx = torch.randperm(N, generator=g)[: N // 100]
    K[:, :, idx] += 3 * Q.mean(dim=(0, 1, 2))
    if heads is not None:
        q_lo, q_hi, kv_lo, kv_hi = heads
        Q, K, V = Q[:, q_lo:q_hi], K[:, kv_lo:kv_hi], V[:, kv_lo:kv_hi]
    if device is not None:
        Q, K, V = Q.to(device), K.to(device), V.to(device)
    if rope:
        Q, K = rope_rotate_half(Q), rope_rotate_half(K)
    if dtype is not None:
        Q, K, V = Q.to(dtype), K.to(dtype), V.to(dtype)
    return Q.contiguous(), K.contiguous(), V.contiguous()
