"""The CPU restatement of the block-granular comparator against golden vectors produced by the
reference's own code (tests/golden/make_golden_block_sparse.py: index builders run as plain
torch, the Triton kernel run by Triton's CPU interpreter in fp16), and the package's index
builders (plain tensor operations, so they run on the CPU too) against both."""
import os

import numpy as np
import pytest
import torch

from oracle.anchor_oracle import make_inputs
from oracle.block_sparse_oracle import (block_sparse_attention_oracle, build_difference_aware_oracle,
                                        build_top_cdf_oracle, build_top_k_oracle)

PATH = os.path.join(os.path.dirname(__file__), "golden", "block_sparse_ref_interp_fp16.npz")
VARIANTS = {
    "top_k3": ("top_k", dict(top_k=3)),
    "diff_t005": ("diff", dict(theta=0.0625, top_k=1000)),
    "diff_t0125_k4": ("diff", dict(theta=0.125, top_k=4)),
    "cdf_05": ("cdf", dict(cdf_threshold=0.5)),
}


@pytest.fixture(scope="module")
def golden():
    g = np.load(PATH)
    Q, K, V = make_inputs(int(g["N"]), int(g["H"]), int(g["H"]), seed=int(g["seed"]), rope=False,
                          dtype=torch.float16, q_shift=0.5)
    return g, Q, K, V


def test_fixture_covers_every_variant(golden):
    g = golden[0]
    assert sorted(g["names"].tolist()) == sorted(VARIANTS)


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_attention_restatement_matches_reference_kernel(golden, name):
    """Same block_index in, the reference kernel's output (every fourth row) out.  The lists hold
    repeated zeros, entries beyond what the kernel reads and entries above the diagonal."""
    g, Q, K, V = golden
    idx = torch.from_numpy(g[f"{name}_index"])
    out = block_sparse_attention_oracle(Q, K, V, idx, mode="fp16")
    err = np.abs(out[0, :, ::4].numpy() - g[f"{name}_out"].astype(np.float32))
    # all but a few elements in ten thousand are bit-identical, the others one fp16 step apart
    assert err.max() <= 1e-3 and err.mean() <= 1e-6 and (err > 0).mean() < 1e-3, (err.max(), err.mean())


def _build_oracle(kind, kw, Qf, Kf):
    sm = Qf.shape[-1] ** -0.5
    if kind == "top_k":
        return build_top_k_oracle(Qf, Kf, kw["top_k"])
    if kind == "cdf":
        idx, ratio = build_top_cdf_oracle(Qf, Kf, kw["cdf_threshold"], sm)
        return idx, ratio, None
    return build_difference_aware_oracle(Qf, Kf, kw["theta"], sm, kw["top_k"])


def _build_package(kind, kw, Qf, Kf):
    from anchor_attention_b200 import block_sparse as bs
    sm = Qf.shape[-1] ** -0.5
    if kind == "top_k":
        return bs.build_block_index(Qf, Kf, kw["top_k"])
    if kind == "cdf":
        return bs.build_block_index_top_cdf(Qf, Kf, kw["cdf_threshold"], 128, 128, sm)
    return bs.build_block_index_difference_aware(Qf, Kf, 128, 128, kw["theta"], sm, kw["top_k"])


def _compare_index(kind, got, ref, extra):
    """Equality wherever the reference's result is determined; elsewhere (entries that depend on
    how topk orders -inf values) the determined part must be contained."""
    got, ref = got.numpy(), ref
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if kind == "top_k":
        det = extra.numpy()
        assert (got[det] == ref[det]).all()
    elif kind == "diff":
        exact = extra.numpy()
        assert (got[exact] == ref[exact]).all()
        for b, h, m in zip(*np.nonzero(~exact)):
            assert set(got[b, h, m].tolist()) - {0} <= set(ref[b, h, m].tolist())
    else:
        assert (got == ref).all()


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_builder_restatements_match_reference_builders(golden, name):
    g, Q, K, _ = golden
    kind, kw = VARIANTS[name]
    idx, ratio, extra = _build_oracle(kind, kw, Q.float(), K.float())
    _compare_index(kind, idx, g[f"{name}_index"], extra)
    assert abs(ratio - float(g[f"{name}_ratio"])) < 1e-9


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_package_builders_match_reference_builders(golden, name):
    """The shipped builders (one scatter instead of the reference's per-row Python loops)."""
    g, Q, K, _ = golden
    kind, kw = VARIANTS[name]
    idx, ratio = _build_package(kind, kw, Q.float(), K.float())
    ref = g[f"{name}_index"]
    assert idx.dtype == torch.int32
    if kind == "top_k":
        _, _, det = build_top_k_oracle(Q.float(), K.float(), kw["top_k"])
        _compare_index(kind, idx, ref, det)
    elif kind == "diff":
        _, _, exact = build_difference_aware_oracle(Q.float(), K.float(), kw["theta"], Q.shape[-1] ** -0.5, kw["top_k"])
        _compare_index(kind, idx, ref, exact)
        # rows that depend on the order of -inf entries in topk: same call, same library, same result
        assert (idx.numpy() == ref).all()
    else:
        _compare_index(kind, idx, ref, None)
    assert abs(ratio - float(g[f"{name}_ratio"])) < 1e-9


def test_package_builders_accept_grouped_kv_heads():
    """K with fewer heads than Q gives the lists the reference builds from the expanded K."""
    from anchor_attention_b200 import block_sparse as bs
    Q, K, _ = make_inputs(1024, 4, 2, seed=3, rope=False, dtype=torch.float32, q_shift=0.5)
    Kx = K.repeat_interleave(2, dim=1)
    a, ra = bs.build_block_index_difference_aware(Q, K, theta=0.0625, sm_scale=128 ** -0.5, top_k=1000)
    b, rb = bs.build_block_index_difference_aware(Q, Kx, theta=0.0625, sm_scale=128 ** -0.5, top_k=1000)
    assert torch.equal(a, b) and ra == rb


def test_dense_lists_give_causal_attention():
    """With every causal block listed the comparator is dense causal attention."""
    from oracle.anchor_oracle import dense_causal_attention
    Q, K, V = make_inputs(512, 2, 1, seed=5, rope=False, dtype=torch.bfloat16)
    nb = 4
    idx = torch.arange(nb, dtype=torch.int32).expand(1, 2, nb, nb).contiguous()
    out = block_sparse_attention_oracle(Q, K, V, idx, mode="fp32")
    dense = dense_causal_attention(Q, K, V)
    assert torch.allclose(out, dense, atol=2e-5)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_scatter_packing_equals_fill_and_sort(seed):
    """The one-scatter packing of the shipped builders against the reference's recipe (zero rows,
    selected indices in the first slots, sort; block_sparse_flash_attention_v2.py:228-239) on
    random masks, empty rows included."""
    from anchor_attention_b200.block_sparse import _pack
    g = torch.Generator().manual_seed(seed)
    B, H, nb = 2, 3, 11
    valid = torch.rand(B, H, nb, nb, generator=g) < 0.3
    valid[0, 0, 0] = False
    valid[1, 2, 5] = True
    width = int(valid.sum(-1).max())
    want = torch.zeros(B, H, nb, width, dtype=torch.int64)
    for b in range(B):
        for h in range(H):
            for m in range(nb):
                sel = torch.arange(nb)[valid[b, h, m]]
                want[b, h, m, :sel.numel()] = sel
    want = want.sort(dim=-1).values.int()
    assert torch.equal(_pack(valid, width), want)
    # a wider row budget only adds leading zeros
    wider = _pack(valid, width + 2)
    assert torch.equal(wider[..., 2:], want) and (wider[..., :2] == 0).all()
