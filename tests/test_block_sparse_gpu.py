"""The block-granular comparator on a B200, through the C ABI, against its CPU restatement.

Tolerance on outputs: max abs <= 2e-2 and mean abs <= 1e-3 in bf16, the bar the operator itself
is held to against the reference's output."""
import os

import numpy as np
import pytest
import torch

from oracle.anchor_oracle import make_inputs
from oracle.block_sparse_oracle import block_sparse_attention_oracle
from parity_util import OUT_MAX_ABS, OUT_MEAN_ABS

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "block_sparse_ref_interp_fp16.npz")
GOLDEN_GPU = os.path.join(os.path.dirname(__file__), "golden", "block_sparse_ref_gpu_bf16.npz")


def _check(out, ref):
    err = (out.float().cpu() - ref).abs()
    assert not torch.isnan(out).any()
    assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS, (float(err.max()), float(err.mean()))


@pytest.mark.parametrize("name", ["top_k3", "diff_t005", "diff_t0125_k4", "cdf_05"])
def test_kernel_matches_oracle_on_the_reference_builders_lists(lib, name):
    """The block lists the reference's builders produced for the golden fixture (zero padding that
    repeats block 0, rows cut off at m + 1 entries, entries above the diagonal), bf16 inputs."""
    from anchor_attention_b200.block_sparse import block_sparse_attend
    g = np.load(GOLDEN)
    Q, K, V = make_inputs(int(g["N"]), int(g["H"]), int(g["H"]), seed=int(g["seed"]), rope=False, q_shift=0.5)
    idx = torch.from_numpy(g[f"{name}_index"])
    ref = block_sparse_attention_oracle(Q, K, V, idx, mode="bf16")
    out = block_sparse_attend(Q.cuda(), K.cuda(), V.cuda(), idx.cuda(), check=True)
    _check(out, ref)


def _random_lists(B, H, nb, width, seed):
    """Ascending rows with repeats and entries above the diagonal; the smallest entry of a row is
    at most the row's own block, so every row attends something."""
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, nb, (B, H, nb, width), generator=g)
    first = (torch.rand(B, H, nb, generator=g) * (torch.arange(nb) + 1)).long()
    idx[..., 0] = first
    return idx.sort(dim=-1).values.int()


def test_grouped_heads_batches_and_token_major_layout(lib):
    """B = 2, 4 query heads on 2 KV heads, q/k/v/out as [B,N,H,D] views, three pairs of query blocks."""
    from anchor_attention_b200.block_sparse import block_sparse_attend
    B, H, Hkv, N = 2, 4, 2, 1536
    qs, ks, vs = [], [], []
    for b in range(B):
        Q, K, V = make_inputs(N, H, Hkv, seed=10 + b, rope=True, q_shift=0.5)
        qs.append(Q); ks.append(K); vs.append(V)
    Q, K, V = torch.cat(qs), torch.cat(ks), torch.cat(vs)
    idx = _random_lists(B, H, N // 128, 5, seed=1)
    ref = block_sparse_attention_oracle(Q, K, V, idx, mode="bf16")
    # token-major storage, handed over as [B,H,N,D] views
    Qt = Q.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    Kt = K.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    Vt = V.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    out_store = torch.zeros(B, N, H, 128, dtype=torch.bfloat16, device="cuda")
    out = block_sparse_attend(Qt, Kt, Vt, idx.cuda(), out=out_store.transpose(1, 2), check=True)
    assert out.data_ptr() == out_store.data_ptr()
    _check(out, ref)
    # a second call on the same inputs gives the same bits
    again = block_sparse_attend(Qt, Kt, Vt, idx.cuda(), check=True)
    assert torch.equal(again, out)


def test_dense_lists_equal_causal_attention(lib):
    """Size-independent property at a larger size: with every causal block listed the comparator
    is dense causal attention.  Checked against the exact fp32 softmax of a row sample; the first
    rows attend a handful of keys and have outputs of magnitude 1-3, whose bf16 rounding alone is
    0.004-0.008, so the mean bound is 2.5e-3 here (the sample is half early rows)."""
    from anchor_attention_b200.block_sparse import block_sparse_attend
    N, H, Hkv = 8192, 8, 2
    Q, K, V = make_inputs(N, H, Hkv, seed=4, rope=True)
    nb = N // 128
    idx = torch.arange(nb, dtype=torch.int32).expand(1, H, nb, nb).contiguous()
    out = block_sparse_attend(Q.cuda(), K.cuda(), V.cuda(), idx.cuda(), check=True).float().cpu()
    rows = torch.tensor([0, 1, 127, 128, 129, 1000, 4095, 4096, 8191])
    sm = 128 ** -0.5
    for h in range(H):
        k, v = K[0, h // (H // Hkv)].float(), V[0, h // (H // Hkv)].float()
        s = (Q[0, h, rows].float() @ k.T) * sm
        s = s.masked_fill(torch.arange(N)[None, :] > rows[:, None], float("-inf"))
        dense = torch.softmax(s, dim=-1) @ v
        err = (out[0, h, rows] - dense).abs()
        assert err.max() <= OUT_MAX_ABS and err.mean() <= 2.5e-3, (float(err.max()), float(err.mean()))


def test_unsorted_list_is_reported(lib):
    from anchor_attention_b200.block_sparse import block_sparse_attend
    Q, K, V = make_inputs(512, 1, 1, seed=0, rope=False)
    idx = torch.tensor([[0, 0, 0], [0, 1, 0], [2, 1, 0], [0, 1, 2]], dtype=torch.int32).view(1, 1, 4, 3)
    with pytest.raises(RuntimeError, match="ascending"):
        block_sparse_attend(Q.cuda(), K.cuda(), V.cuda(), idx.cuda(), check=True)
    # the context is intact: a proper call works
    idx = torch.tensor([[0, 0, 0], [0, 0, 1], [0, 1, 2], [1, 2, 3]], dtype=torch.int32).view(1, 1, 4, 3)
    out = block_sparse_attend(Q.cuda(), K.cuda(), V.cuda(), idx.cuda(), check=True)
    _check(out, block_sparse_attention_oracle(Q, K, V, idx, mode="bf16"))


@pytest.mark.parametrize("L,mode,kw", [(1900, "top_k", dict(top_k=4)),            # 15 blocks: an odd count
                                       (2000, "top_cdf", dict(top_k=4, cdf_threshold=0.5)),
                                       (2000, "top_difference_aware", dict(top_k=6, theta=0.0625)),
                                       (1900, "top_difference_aware", dict(top_k=1000, theta=0.0625))])
def test_wrapper_pads_builds_and_attends(lib, L, mode, kw):
    """The reference-facing call on a length that is not a multiple of the block: the lists built on
    the device are valid (ascending, in range), the output equals the restatement's on those
    lists, and the ratio is the reference's formula."""
    from anchor_attention_b200 import block_sparse as bs
    H, Hkv = 4, 2
    Q, K, V = make_inputs(2048, H, Hkv, seed=6, rope=True, q_shift=0.5)
    Q, K, V = Q[:, :, :L].contiguous(), K[:, :, :L].contiguous(), V[:, :, :L].contiguous()
    out, ratio = bs.block_sparse_attention(Q.cuda(), K.cuda(), V.cuda(), mode=mode, return_sparsity_ratio=True, **kw)
    assert out.shape == (1, H, L, 128) and 0.0 < ratio <= 1.0
    # the same steps by hand: pad, build on the device, restate on the CPU
    pad = (-L) % 128
    Qp, Kp, Vp = (torch.nn.functional.pad(t, (0, 0, 0, pad)) for t in (Q, K, V))
    sm = 128 ** -0.5
    if mode == "top_k":
        idx, r2 = bs.build_block_index(Qp.cuda(), Kp.cuda(), kw["top_k"])
    elif mode == "top_cdf":
        idx, r2 = bs.build_block_index_top_cdf(Qp.cuda(), Kp.cuda(), kw["cdf_threshold"], 128, 128, sm)
    else:
        idx, r2 = bs.build_block_index_difference_aware(Qp.cuda(), Kp.cuda(), 128, 128, kw["theta"], sm, kw["top_k"])
    assert r2 == ratio
    idx = idx.cpu()
    nb = Qp.shape[2] // 128
    assert idx.shape[:3] == (1, H, nb) and idx.min() >= 0 and idx.max() < nb
    assert (idx[..., 1:] >= idx[..., :-1]).all()
    ref = block_sparse_attention_oracle(Qp, Kp, Vp, idx, mode="bf16")[:, :, :L]
    _check(out, ref)


@pytest.mark.skipif(not os.path.exists(GOLDEN_GPU), reason="no bf16 fixture of the reference kernel")
@pytest.mark.parametrize("name", ["top_k3", "diff_t005", "diff_t0125_k4", "cdf_05"])
def test_kernel_matches_reference_kernel_run_on_gpu(lib, name):
    """Against the reference's compiled Triton kernel (bf16, run on a B200; every fourth row kept)."""
    from anchor_attention_b200.block_sparse import block_sparse_attend
    g = np.load(GOLDEN_GPU)
    Q, K, V = make_inputs(int(g["N"]), int(g["H"]), int(g["H"]), seed=int(g["seed"]), rope=False, q_shift=0.5)
    idx = torch.from_numpy(g[f"{name}_index"])
    out = block_sparse_attend(Q.cuda(), K.cuda(), V.cuda(), idx.cuda(), check=True)
    ref = torch.from_numpy(g[f"{name}_out"]).view(torch.bfloat16).float()
    _check(out[0, :, ::4], ref)
