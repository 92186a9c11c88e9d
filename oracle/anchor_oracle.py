"""CPU restatement of the reference's anchor-attention prefill operator.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared
with; nothing in the shipped package imports it.  Only the test-suite, the
smoke entry and the benchmark's CPU-baseline legs may call it.

What it restates (paths are relative to the reference project's root):

* operator entry and orchestration ........ anchor_attn/src/ops/anchor_attn_v4.py:226-273, 291-324
* step 1, anchor / window attention ....... anchor_attn/src/ops/anchor_step_1_2_v2.py:8-161
* step 2, stripe identification ........... anchor_attn/src/ops/get_mask_test.py:7-124
  (cross-checked with the reference's own dense restatement, get_mask_test.py:162-232)
* step 3, gathered sparse flash attention . anchor_attn/src/ops/anchor_attn_v4.py:7-105
* GQA head mapping (repeat_kv order) ...... my_utils/ops_util.py:6-24

Pinning status: the reference ships no golden vectors or assertions for this
path.  The restatement is pinned against outputs of the reference's own Triton
kernels executed here in the Triton CPU interpreter (fp16 only; the interpreter
has no bf16), see tests/golden/make_golden.py; the committed fixtures hold those
outputs.  The bf16 mode is the same code with a different rounding type.

Three arithmetic modes, selected by ``mode``:
  "bf16" / "fp16" : every point where the reference kernels round to the input
                    dtype is an explicit round-trip through that dtype; all
                    other arithmetic is fp32.
  "fp32"          : no rounding at all, exact scale constants.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

LOG2E = 1.44269504  # the literal the reference kernels use

_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": None}


def _rounder(mode: str):
    dt = _DT[mode]
    if dt is None:
        return lambda x: x
    return lambda x: x.to(dt).to(torch.float32)


def f32(x: float) -> float:
    """Value of a Python double after conversion to fp32."""
    return float(torch.tensor(x, dtype=torch.float32))


# --------------------------------------------------------------------------
# query pre-scaling
# --------------------------------------------------------------------------
def scale_q_step1(q: torch.Tensor, sm_scale: float, mode: str) -> torch.Tensor:
    """anchor_step_1_2_v2.py:115-116.  ``sm_scale`` and the log2(e) literal are
    compile-time constants there, so both are materialised in the tensor's
    dtype and the product is rounded after each multiply."""
    rd = _rounder(mode)
    q = q.to(torch.float32)
    if mode == "fp32":
        return q * f32(sm_scale) * f32(LOG2E)
    c1 = rd(torch.tensor(sm_scale, dtype=torch.float32))
    c2 = rd(torch.tensor(LOG2E, dtype=torch.float32))
    return rd(rd(q * c1) * c2)


def scale_q_step3(q: torch.Tensor, sm_scale: float, mode: str) -> torch.Tensor:
    """anchor_attn_v4.py:65-66.  ``sm_scale`` is a run-time fp32 argument here:
    two fp32 multiplies, then one rounding."""
    rd = _rounder(mode)
    return rd(q.to(torch.float32) * f32(sm_scale) * f32(LOG2E))


# --------------------------------------------------------------------------
# step 1
# --------------------------------------------------------------------------
def step1(q, k, v, sm_scale, block_size=128, step=16, mode="bf16", blocks=None):
    """Window attention over the first ``block_size*step`` keys plus the query's
    own big block, causal.  q [N,D] of one head; k, v [N,D] of its KV head.
    Returns (M [N], L [N], Acc [N,D]) fp32, M in the log2 domain.
    Follows anchor_step_1_2_v2.py:119-161 (tile-by-tile online softmax with an
    additive -1e6 mask); tiles that are masked out entirely leave the running
    state unchanged bit for bit and are skipped.  ``blocks`` restricts the work
    to the query rows of those big blocks (other rows are left at NaN)."""
    rd = _rounder(mode)
    N, D = q.shape
    T = 128  # BLOCK_SZ_M == BLOCK_SZ_N in the reference's launch (anchor_attn_v4.py:232)
    G = block_size * step
    qs = scale_q_step1(q, sm_scale, mode)
    kf = k.to(torch.float32)
    vf = v.to(torch.float32)
    M = torch.full((N,), float("nan"), dtype=torch.float32)
    L = torch.full((N,), float("nan"), dtype=torch.float32)
    Acc = torch.full((N, D), float("nan"), dtype=torch.float32)
    ar = torch.arange(T)
    for qb in range(N // T):
        rows = slice(qb * T, (qb + 1) * T)
        b = (qb * T) // G
        if blocks is not None and b not in blocks:
            continue
        init_end = min(G, (qb + 1) * T)
        local_start = max(b * G, init_end)
        tiles = list(range(0, init_end, T)) + list(range(local_start, (qb + 1) * T, T))
        qt = qs[rows]
        m_i = torch.full((T,), -float("inf"))
        l_i = torch.zeros(T)
        acc = torch.zeros(T, D)
        offs_m = qb * T + ar
        for j in tiles:
            s = qt @ kf[j:j + T].T
            causal = (ar[None, :] + j) <= offs_m[:, None]
            s = s + torch.where(causal, 0.0, -1e6)
            m_new = torch.maximum(m_i, s.max(dim=1).values)
            p = torch.exp2(s - m_new[:, None])
            alpha = torch.exp2(m_i - m_new)
            l_i = l_i * alpha + p.sum(dim=1)
            acc = acc * alpha[:, None] + rd(p) @ vf[j:j + T]
            m_i = m_new
        M[rows], L[rows], Acc[rows] = m_i, l_i, acc
    return M, L, Acc


# --------------------------------------------------------------------------
# step 2
# --------------------------------------------------------------------------
def _tree_sum_rows(x: torch.Tensor, rd) -> torch.Tensor:
    """Sum the rows of ``x`` [..., BS, C] (BS = 64, 128 or 256) in the order the compiled
    reference kernel uses on the GPU for BS = 128: row r sits in lane r%32 of warp r//32;
    each group of 32 rows is reduced with xor-butterflies at 16, 8, 4, 2, 1; the BS/32 group
    sums are combined by halving as well (four groups: (W0+W2)+(W1+W3)).  Every add is rounded
    by ``rd``.  For BS = 64 and 256 this is the order of the CUDA pooling kernel; the order of
    the reference's compiled reduction at those sizes has not been derived."""
    bs = x.shape[-2]
    assert bs in (64, 128, 256)
    w = x.reshape(*x.shape[:-2], bs // 32, 32, x.shape[-1])
    for half in (16, 8, 4, 2, 1):
        w = rd(w[..., :half, :] + w[..., half:2 * half, :])
    w = w[..., 0, :]                      # [..., BS/32, C]
    half = bs // 64
    while half >= 1:
        w = rd(w[..., :half, :] + w[..., half:2 * half, :])
        half //= 2
    return w[..., 0, :]


def _seq_sum_rows(x: torch.Tensor, rd) -> torch.Tensor:
    """Plain left-to-right sum over the 128 rows, rounding after each add (the
    order the Triton CPU interpreter's numpy reduction produces)."""
    acc = x[..., 0, :]
    for r in range(1, x.shape[-2]):
        acc = rd(acc + x[..., r, :])
    return acc


def pool_q(q: torch.Tensor, block_size: int, mode: str, order: str = "tree") -> torch.Tensor:
    """get_mask_test.py:75-78: per-block mean of q, the sum carried in the input
    dtype, the division in fp32, the result rounded to the input dtype."""
    rd = _rounder(mode)
    N, D = q.shape
    x = q.to(torch.float32).reshape(N // block_size, block_size, D)
    if order == "tree" and block_size in (64, 128, 256):
        s = _tree_sum_rows(x, rd)
    elif order == "seq":
        s = _seq_sum_rows(x, rd)
    else:
        s = _seq_sum_rows(x, rd)
    return rd(s / block_size)


def pool_anchor(M: torch.Tensor, block_size: int, mode: str, order: str = "tree") -> torch.Tensor:
    """get_mask_test.py:81-84: fp32 mean of the step-1 row maxima per block,
    rounded to the input dtype."""
    rd = _rounder(mode)
    x = M.reshape(-1, block_size, 1)
    if order == "tree" and block_size in (64, 128, 256):
        s = _tree_sum_rows(x, lambda t: t)[..., 0]
    else:
        s = x.sum(dim=1)[..., 0]
    return rd(s / block_size)


def step2(q, k, M, sm_scale, theta, block_size=128, step=16, mode="bf16", order="tree",
          return_margin: bool = False, diff_add: str = "fp32", blocks=None):
    """Difference-aware stripe identification for one head.
    Returns a list (one entry per big block) of ascending int32 column ids.
    Follows get_mask_test.py:86-124: candidates of big block b are the columns
    [block_size, b*G - block_size); a column is kept when, for any of the
    ``step`` pooled rows, rounded(pooled_q.k * scale) + theta*log2e >= pooled anchor,
    the add and the compare in fp32.

    ``diff_add`` = "input" reproduces an artefact of Triton's CPU interpreter,
    which treats the run-time ``diff`` argument as a weak Python scalar, so the add
    is rounded to the input dtype; the compiled GPU kernel receives ``diff`` as an
    fp32 argument and adds in fp32 ("fp32", the default).

    With ``return_margin`` also returns, per big block, the fp32 value
    max_r(score + diff - anchor) per candidate column before the score is
    rounded and its rounding half-width, which tests use to build the tie band.
    """
    rd = _rounder(mode)
    N, D = q.shape
    G = block_size * step
    NB = N // G
    qp = pool_q(q, block_size, mode, order)            # [N/bs, D]
    ap = pool_anchor(M, block_size, mode, order)       # [N/bs]
    kf = k.to(torch.float32)
    qk_scale = f32(sm_scale * LOG2E)                   # python-double product, then fp32
    diff = f32(theta * LOG2E)                          # anchor_attn_v4.py:298, passed as an fp32 argument
    ids: List[torch.Tensor] = []
    margins = []
    for b in range(NB):
        lo, hi = block_size, b * G - block_size
        if hi <= lo or (blocks is not None and b not in blocks):
            ids.append(torch.empty(0, dtype=torch.int32))
            margins.append(None)
            continue
        raw = (qp[b * step:(b + 1) * step] @ kf[lo:hi].T) * qk_scale   # [step, C] fp32
        sc = rd(raw)
        a = ap[b * step:(b + 1) * step, None]
        if diff_add == "input":
            hit = (rd(sc + rd(torch.tensor(diff))) >= a).any(dim=0)
        else:
            hit = ((sc + diff) >= a).any(dim=0)
        ids.append((torch.nonzero(hit)[:, 0] + lo).to(torch.int32))
        if return_margin:
            margins.append((raw + diff - a, raw.abs()))
    if return_margin:
        return ids, margins
    return ids


def step2_dense_check(q, k, M, sm_scale, theta, block_size=128, step=16):
    """The reference's own dense formulation (get_mask_test.py:162-232) in fp32:
    mean-pooled q against all keys, OR over ``step`` pooled rows, then the
    candidate range cut.  Used only to cross-check ``step2`` in fp32 mode."""
    N, D = q.shape
    G = block_size * step
    mq = q.float().reshape(-1, block_size, D).mean(dim=1)
    ma = M.reshape(-1, block_size).mean(dim=1, keepdim=True)
    att = (mq @ (k.float().T * f32(sm_scale * LOG2E)) + f32(theta * LOG2E)) >= ma
    blk = att.reshape(-1, step, N).any(dim=1)
    out = []
    for i in range(N // G):
        end = i * G - block_size
        if end <= block_size:
            out.append(torch.empty(0, dtype=torch.int32))
        else:
            out.append((torch.nonzero(blk[i, block_size:end])[:, 0] + block_size).to(torch.int32))
    return out


# --------------------------------------------------------------------------
# step 3
# --------------------------------------------------------------------------
def step3(q, k, v, ids, M, L, Acc, sm_scale, block_size=128, step=16, mode="bf16", blocks=None):
    """Continue the online softmax of step 1 over the selected columns, 128 ids
    at a time (anchor_attn_v4.py:62-105).  The 16 query blocks of a big block
    share one id list, so they are processed together; per-row arithmetic is
    identical to the reference's per-128-row programs."""
    rd = _rounder(mode)
    N, D = q.shape
    G = block_size * step
    qs = scale_q_step3(q, sm_scale, mode)
    kf = k.to(torch.float32)
    vf = v.to(torch.float32)
    out = torch.full((N, D), float("nan"), dtype=torch.float32)
    for b in range(N // G):
        if blocks is not None and b not in blocks:
            continue
        rows = slice(b * G, (b + 1) * G)
        m_i, l_i, acc = M[rows].clone(), L[rows].clone(), Acc[rows].clone()
        idb = ids[b].long()
        for c0 in range(0, idb.numel(), 128):
            sel = idb[c0:c0 + 128]
            s = qs[rows] @ kf[sel].T
            m_new = torch.maximum(m_i, s.max(dim=1).values)
            alpha = torch.exp2(m_i - m_new)
            p = torch.exp2(s - m_new[:, None])
            acc = acc * alpha[:, None] + rd(p) @ vf[sel]
            l_i = l_i * alpha + p.sum(dim=1)
            m_i = m_new
        out[rows] = acc / l_i[:, None]
    return rd(out)


# --------------------------------------------------------------------------
# whole operator
# --------------------------------------------------------------------------
@dataclass
class OracleResult:
    out: torch.Tensor                       # [B,H,N,D] fp32 (already rounded to the mode's dtype)
    ids: List[List[List[torch.Tensor]]]     # [B][H][NB] ascending int32 column ids
    counts: torch.Tensor                    # [B,H,NB] int32
    M: torch.Tensor                         # [B,H,N]
    L: torch.Tensor                         # [B,H,N]
    Acc: Optional[torch.Tensor]             # [B,H,N,D] (None unless keep_state)
    ratio: float


def anchor_attn_oracle(Q, K, V, sm_scale=None, block_size=128, step=16, difference=12.0,
                       mode="bf16", order="tree", keep_state=True, diff_add="fp32") -> OracleResult:
    """Restatement of ``anchor_attn`` (anchor_attn_v4.py:291-324).  Q [B,H,N,D];
    K, V [B,Hkv,N,D] with Hkv dividing H; query head h reads KV head
    h // (H/Hkv), the order ``repeat_kv`` produces (my_utils/ops_util.py:6-24).
    ``difference`` is theta in natural-log units, as the reference takes it."""
    assert step in (16, 32), f"Invalid step size: {step}. Only step sizes 16 or 32 are supported."
    B, H, N, D = Q.shape
    Hkv = K.shape[1]
    assert H % Hkv == 0
    G = block_size * step
    assert N % G == 0, f"Sequence length {N} must be divisible by (block_size * step = {G})."
    sm_scale = sm_scale if sm_scale else 1.0 / (D ** 0.5)
    NB = N // G
    out = torch.empty(B, H, N, D, dtype=torch.float32)
    Ms = torch.empty(B, H, N)
    Ls = torch.empty(B, H, N)
    Accs = torch.empty(B, H, N, D) if keep_state else None
    counts = torch.zeros(B, H, NB, dtype=torch.int32)
    all_ids = []
    for z in range(B):
        ids_z = []
        for h in range(H):
            kv = h // (H // Hkv)
            q, k, v = Q[z, h], K[z, kv], V[z, kv]
            M, L, Acc = step1(q, k, v, sm_scale, block_size, step, mode)
            ids = step2(q, k, M, sm_scale, difference, block_size, step, mode, order, diff_add=diff_add)
            out[z, h] = step3(q, k, v, ids, M, L, Acc, sm_scale, block_size, step, mode)
            Ms[z, h], Ls[z, h] = M, L
            if keep_state:
                Accs[z, h] = Acc
            for b in range(NB):
                counts[z, h, b] = ids[b].numel()
            ids_z.append(ids)
        all_ids.append(ids_z)
    ratio = float(counts.sum()) / ((B * H * N * N / (block_size * step)) // 2)   # anchor_attn_v4.py:271
    return OracleResult(out, all_ids, counts, Ms, Ls, Accs, ratio)


def oracle_big_blocks(q, k, v, blocks, sm_scale=None, block_size=128, step=16, difference=12.0,
                      mode="bf16", order="tree"):
    """Everything the operator computes for the query rows of the given big
    blocks of ONE head (q [N,D]; k, v [N,D] of its KV head): used to check
    full-size problems on a sample of blocks.  Returns (M, L, Acc, ids, out) with
    rows outside ``blocks`` left at NaN / empty."""
    D = q.shape[-1]
    sm_scale = sm_scale if sm_scale else 1.0 / (D ** 0.5)
    M, L, Acc = step1(q, k, v, sm_scale, block_size, step, mode, blocks=blocks)
    ids = step2(q, k, torch.nan_to_num(M), sm_scale, difference, block_size, step, mode, order, blocks=blocks)
    out = step3(q, k, v, ids, M, L, Acc, sm_scale, block_size, step, mode, blocks=blocks)
    return M, L, Acc, ids, out


def dense_causal_attention(Q, K, V, sm_scale=None) -> torch.Tensor:
    """Plain fp32 causal softmax attention with the same GQA mapping; the
    comparator for recall figures (definition: ops_profile_v2.py:514-532)."""
    B, H, N, D = Q.shape
    Hkv = K.shape[1]
    sm_scale = sm_scale if sm_scale else 1.0 / (D ** 0.5)
    out = torch.empty(B, H, N, D)
    mask = torch.ones(N, N, dtype=torch.bool).tril()
    for z in range(B):
        for h in range(H):
            kv = h // (H // Hkv)
            s = (Q[z, h].float() @ K[z, kv].float().T) * sm_scale
            s = s.masked_fill(~mask, -float("inf"))
            out[z, h] = torch.softmax(s, dim=-1) @ V[z, kv].float()
    return out


# --------------------------------------------------------------------------
# synthetic inputs shared by tests and the benchmark's CPU legs
# --------------------------------------------------------------------------
def rope_rotate_half(x: torch.Tensor, base: float = 500000.0) -> torch.Tensor:
    """HF rotate-half RoPE over positions 0..N-1, fp32.  x [..., N, D]."""
    N, D = x.shape[-2:]
    inv = base ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    ang = torch.arange(N, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    cos, sin = emb.cos(), emb.sin()
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return x * cos + torch.cat([-x2, x1], dim=-1) * sin


def make_inputs(N, H, Hkv, D=128, seed=0, rope=True, dtype=torch.bfloat16, q_shift=0.0):
    """Seeded synthetic Q/K/V: N(0,1) entries, the first 64 key rows scaled by 4
    (attention sink), a random 1 % of key positions shifted by 3*mean(Q)
    (vertical stripes), optional RoPE at base 500000, then a cast to ``dtype``.
    ``q_shift`` adds a constant to Q before the stripes are made (a labelled
    auxiliary distribution that exercises the sparse regime)."""
    g = torch.Generator("cpu").manual_seed(seed)
    Q = torch.randn(1, H, N, D, generator=g)
    K = torch.randn(1, Hkv, N, D, generator=g)
    V = torch.randn(1, Hkv, N, D, generator=g)
    if q_shift:
        Q = Q + q_shift
    K[:, :, :64] *= 4
    idx = torch.randperm(N, generator=g)[: N // 100]
    K[:, :, idx] += 3 * Q.mean(dim=(0, 1, 2))
    if rope:
        Q, K = rope_rotate_half(Q), rope_rotate_half(K)
    if dtype is not None:
        Q, K, V = Q.to(dtype), K.to(dtype), V.to(dtype)
    return Q, K, V
