"""CPU restatement of the reference's block-granular comparator.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared
with; nothing in the shipped package imports it.

What it restates (paths are relative to the reference project's root):

* the block-sparse flash-attention kernel ... anchor_attn/src/ops/block_sparse_flash_attention_v2.py:10-110
* the three index builders .................. the same file, :150-190 (top_k), :193-243 (top_cdf),
                                               :246-309 (top_difference_aware)
* the wrapper (padding, sm_scale) ........... the same file, :311-356

Pinning status: the reference has no golden vectors for this path.  The restatement is
pinned against the reference's own functions run here -- the index builders as plain torch
on the CPU, the Triton kernel in the Triton CPU interpreter (fp16 only) -- see
tests/golden/make_golden_block_sparse.py; the committed fixture holds their outputs.

The builders are written row by row on purpose (small cases only); where the reference's
result depends on how ``torch.topk`` orders equal values (rows with fewer causally valid
blocks than ``top_k``), the ambiguous entries are listed separately: they lie beyond the
entries the kernel reads, or are causally masked for every row, and change no output.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from .anchor_oracle import LOG2E, _rounder, f32

BLOCK = 128


def block_sparse_attention_oracle(q, k, v, block_index, sm_scale=None, mode="bf16") -> torch.Tensor:
    """block_sparse_flash_attention_v2.py:10-110 for seqlen == N.  q [B,H,N,D]; k, v [B,Hkv,N,D]
    (query head h reads KV head h // (H // Hkv)); block_index integer [B,H,N/128,MAX].
    Query block m walks the first min(m + 1, MAX) entries of its row (:66) in order, duplicates
    included; scores of keys after the query row are -inf (:76-77).  Returns fp32 values that
    are exactly representable in the rounding type of ``mode``."""
    rd = _rounder(mode)
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    sm = (D ** -0.5) if sm_scale is None else sm_scale
    qk_scale = f32(f32(sm) * f32(LOG2E))                    # :58, fp32 scalar arithmetic in the kernel
    out = torch.empty(B, H, N, D, dtype=torch.float32)
    ar = torch.arange(BLOCK)
    max_blocks = block_index.shape[-1]
    for b in range(B):
        for h in range(H):
            kf = k[b, h // (H // Hkv)].to(torch.float32)
            vf = v[b, h // (H // Hkv)].to(torch.float32)
            qs = rd(q[b, h].to(torch.float32) * qk_scale)   # :61-62
            for m in range(N // BLOCK):
                rows = slice(m * BLOCK, (m + 1) * BLOCK)
                offs_m = m * BLOCK + ar
                m_i = torch.full((BLOCK,), -float("inf"))
                l_i = torch.zeros(BLOCK)
                acc = torch.zeros(BLOCK, D)
                for e in range(min(m + 1, max_blocks)):
                    blk = int(block_index[b, h, m, e])
                    cols = blk * BLOCK + ar
                    s = qs[rows] @ kf[cols].T
                    s = torch.where(cols[None, :] <= offs_m[:, None], s, torch.full_like(s, -float("inf")))
                    m_new = torch.maximum(m_i, s.max(dim=1).values)
                    alpha = torch.exp2(m_i - m_new)
                    p = torch.exp2(s - m_new[:, None])
                    acc = acc * alpha[:, None] + rd(p) @ vf[cols]
                    l_i = l_i * alpha + p.sum(dim=1)
                    m_i = m_new
                out[b, h, rows] = rd(acc / l_i[:, None])
    return out


def dense_causal_tail_oracle(q, k, v, sm_scale=None, mode="bf16") -> torch.Tensor:
    """Dense causal attention of the LAST Nq positions of an Nkv-long sequence with the arithmetic
    of the block kernel above: q [B,H,Nq,D], k/v [B,Hkv,Nkv,D]; row i sits at position
    Nkv - Nq + i and attends keys 0 .. Nkv - Nq + i.  The semantics of the reference's dense calls
    for the prefill tail and later chunks (anchor_attn/src/modules/llama/anchor_attention.py:76-88,
    101-113, which go to flash-attn with causal=True, bottom-right aligned; flash-attn's own
    arithmetic is not pinned by anything in the reference).  Rounding points as in the block
    kernel: scaled queries and probabilities rounded to the input type, everything else fp32;
    128-row query tiles counted from the first tail row, 128-key blocks in ascending order."""
    rd = _rounder(mode)
    B, H, Nq, D = q.shape
    Hkv, Nkv = k.shape[1], k.shape[2]
    off = Nkv - Nq
    sm = (D ** -0.5) if sm_scale is None else sm_scale
    qk_scale = f32(f32(sm) * f32(LOG2E))
    out = torch.empty(B, H, Nq, D, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            kf = k[b, h // (H // Hkv)].to(torch.float32)
            vf = v[b, h // (H // Hkv)].to(torch.float32)
            qs = rd(q[b, h].to(torch.float32) * qk_scale)
            for r0 in range(0, Nq, BLOCK):
                r1 = min(Nq, r0 + BLOCK)
                pos = off + torch.arange(r0, r1)
                m_i = torch.full((r1 - r0,), -float("inf"))
                l_i = torch.zeros(r1 - r0)
                acc = torch.zeros(r1 - r0, D)
                for c0 in range(0, int(pos[-1]) + 1, BLOCK):
                    c1 = min(Nkv, c0 + BLOCK)
                    cols = torch.arange(c0, c1)
                    s = qs[r0:r1] @ kf[c0:c1].T
                    s = torch.where(cols[None, :] <= pos[:, None], s, torch.full_like(s, -float("inf")))
                    m_new = torch.maximum(m_i, s.max(dim=1).values)
                    alpha = torch.exp2(m_i - m_new)
                    p = torch.exp2(s - m_new[:, None])
                    acc = acc * alpha[:, None] + rd(p) @ vf[c0:c1]
                    l_i = l_i * alpha + p.sum(dim=1)
                    m_i = m_new
                out[b, h, r0:r1] = rd(acc / l_i[:, None])
    return out


def _pooled_scores(query, key, scale):
    """Block means (in the input dtype, as ``Tensor.mean`` gives them), optional scale, scores
    of block means, -inf above the diagonal (:166-174)."""
    B, H, N, D = query.shape
    nb = N // BLOCK
    qp = query.view(B, H, nb, BLOCK, D).mean(dim=-2)
    if scale is not None:
        qp = qp * scale
    kp = key.view(B, H, nb, BLOCK, D).mean(dim=-2)
    p = torch.einsum('bhmk,bhnk->bhmn', qp, kp)
    for m in range(nb):
        p[:, :, m, m + 1:] = -float("inf")
    return p


def _pack_rows(rows: List[List[int]], shape, width: int) -> torch.Tensor:
    """Zero-initialised rows, the selected indices in the first slots, then sorted (:228-239)."""
    B, H, nb = shape
    out = torch.zeros(B, H, nb, width, dtype=torch.int64)
    it = iter(rows)
    for b in range(B):
        for h in range(H):
            for m in range(nb):
                sel = next(it)
                out[b, h, m, :len(sel)] = torch.tensor(sel[:width], dtype=torch.int64)
    return out.sort(dim=-1).values.int()


def build_top_k_oracle(query, key, top_k: int) -> Tuple[torch.Tensor, float, torch.Tensor]:
    """:150-190.  Returns (block_index, ratio, determined) where ``determined`` [B,H,nb,k] marks
    the entries that do not depend on the order ``torch.topk`` gives equal (-inf) values: all
    of a row with at least k causally valid blocks, and the first m + 1 entries (0..m) of an
    earlier row -- which are the only ones the kernel reads there."""
    B, H, N, _ = query.shape
    nb = N // BLOCK
    p = _pooled_scores(query, key, None)
    top_k = min(int(top_k), nb)
    idx = torch.zeros(B, H, nb, top_k, dtype=torch.int32)
    det = torch.zeros(B, H, nb, top_k, dtype=torch.bool)
    for b in range(B):
        for h in range(H):
            for m in range(nb):
                order = sorted(range(m + 1), key=lambda n: (-float(p[b, h, m, n]), n))
                if m + 1 >= top_k:
                    idx[b, h, m] = torch.tensor(sorted(order[:top_k]), dtype=torch.int32)
                    det[b, h, m] = True
                else:
                    # all m + 1 valid blocks, then blocks from above the diagonal in an unspecified order
                    idx[b, h, m, :m + 1] = torch.arange(m + 1, dtype=torch.int32)
                    det[b, h, m, :m + 1] = True
                    idx[b, h, m, m + 1:] = torch.arange(m + 1, top_k, dtype=torch.int32)
    total_possible = B * H * nb * (nb + 1) // 2
    total_used = B * H * ((nb - top_k) * top_k + top_k * (top_k + 1) // 2)
    return idx, (total_used / total_possible if total_possible else 0.0), det


def build_top_cdf_oracle(query, key, cdf_threshold: float, sm_scale: float) -> Tuple[torch.Tensor, float]:
    """:193-243: the first ``cutoff`` blocks of each row, cutoff = 1 + the first position where
    the running sum of the row's softmax exceeds the threshold (0 if it never does)."""
    B, H, N, _ = query.shape
    nb = N // BLOCK
    p = _pooled_scores(query, key, sm_scale)
    cdf = torch.softmax(p, dim=-1).cumsum(dim=-1)
    rows, used = [], 0
    for b in range(B):
        for h in range(H):
            for m in range(nb):
                over = [n for n in range(nb) if float(cdf[b, h, m, n]) > cdf_threshold]
                cutoff = (over[0] if over else 0) + 1
                sel = [n for n in range(nb) if n < cutoff and n <= m]
                rows.append(sel)
                used += len(sel)
    width = max(len(r) for r in rows)
    total_possible = B * H * nb * (nb + 1) // 2
    return _pack_rows(rows, (B, H, nb), width), (used / total_possible if total_possible else 0.0)


def build_difference_aware_oracle(query, key, theta: float, sm_scale: float, top_k: int):
    """:246-309.  Returns (block_index, ratio, exact): ``exact`` is False for a row whose result
    depends on how ``torch.topk`` orders -inf entries (fewer than ``top_k`` blocks pass the
    test while ``top_k`` clips, :285-289); for such a row the passing blocks are returned,
    left-padded with zeros like the unclipped rows."""
    B, H, N, _ = query.shape
    nb = N // BLOCK
    top_k = int(top_k)
    p = _pooled_scores(query, key, sm_scale)
    rows, exact, used = [], [], 0
    for b in range(B):
        for h in range(H):
            for m in range(nb):
                sc = [float(p[b, h, m, n]) for n in range(m + 1)]
                best = max(sc)
                arg = sc.index(best)
                # the difference and the comparison are made in the tensor's dtype (:276-277)
                passes = (p[b, h, m, arg] - p[b, h, m, :m + 1]) <= theta
                sel = [n for n in range(m + 1) if bool(passes[n]) or n == arg]
                ok = True
                if top_k < nb:
                    if len(sel) >= top_k:
                        sel = sorted(sorted(sel, key=lambda n: (-sc[n], n))[:top_k])
                    else:
                        ok = False
                    used += top_k
                else:
                    used += len(sel)
                rows.append(sel)
                exact.append(ok)
    width = min(max(len(r) for r in rows), top_k) if top_k >= nb else top_k
    total_possible = B * H * nb * (nb + 1) // 2
    return (_pack_rows(rows, (B, H, nb), width), (used / total_possible if total_possible else 0.0),
            torch.tensor(exact).view(B, H, nb))
