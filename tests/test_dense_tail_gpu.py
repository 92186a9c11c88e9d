"""Dense causal attention of the last q positions over kv keys on the library's own kernel
(the tail of a prefill, a later prefill chunk), through the C ABI.

Checked against the CPU restatement with the kernel's rounding points (scaled queries and
probabilities rounded to bf16): max 2e-2 / mean 1e-3, the operator's tolerance; and against exact
fp32 dense softmax on the same bf16 inputs, where those two roundings show: max 5e-2 / mean 3e-3."""
import pytest
import torch

from oracle.anchor_oracle import dense_causal_attention as dense_oracle, make_inputs
from oracle.block_sparse_oracle import dense_causal_tail_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nq,nkv,H,Hkv", [
    (333, 4096 + 333, 4, 2),       # the tail of a prefill whose length is not a multiple of 2048
    (2048, 6144, 2, 1),            # a later prefill chunk
    (77, 77, 2, 2),                # a short prompt: everything dense, offset 0
    (1000, 1000, 7, 1),            # group of seven, rows and keys both ragged
    (16, 5000, 2, 1),              # few queries, many keys (keys not a multiple of 128)
    (512, 640, 2, 1),              # offset 128: the diagonal falls on a block boundary
])
def test_dense_tail_matches_dense_softmax(lib, nq, nkv, H, Hkv):
    from anchor_attention_b200 import dense_causal_attention
    n = ((nkv + 127) // 128) * 128
    Q, K, V = make_inputs(max(n, 2048), H, Hkv, seed=nq, rope=True)
    Q, K, V = Q[:, :, nkv - nq:nkv], K[:, :, :nkv], V[:, :, :nkv]
    got = dense_causal_attention(Q.cuda().contiguous(), K.cuda().contiguous(), V.cuda().contiguous())
    assert got.shape == (1, H, nq, 128)
    err = (got.float().cpu() - dense_causal_tail_oracle(Q, K, V)).abs()
    assert err.max() <= 2e-2 and err.mean() <= 1e-3, (float(err.max()), float(err.mean()))
    exact = dense_oracle(torch.cat([torch.zeros(1, H, nkv - nq, 128, dtype=Q.dtype), Q], dim=2), K, V)[:, :, nkv - nq:]
    err = (got.float().cpu() - exact).abs()
    assert err.max() <= 5e-2 and err.mean() <= 3e-3, (float(err.max()), float(err.mean()))


def test_dense_tail_strided_views_and_token_major_output(lib):
    """[B,N,H,D] memory for q/k/v and a token-major output view, as the model hook passes them."""
    from anchor_attention_b200 import dense_causal_attention
    nq, nkv, H, Hkv = 300, 2348, 4, 2
    Q, K, V = make_inputs(4096, H, Hkv, seed=5, rope=True)
    Q, K, V = Q[:, :, nkv - nq:nkv].cuda(), K[:, :, :nkv].cuda(), V[:, :, :nkv].cuda()
    base = dense_causal_attention(Q.contiguous(), K.contiguous(), V.contiguous())
    Qs, Ks, Vs = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (Q, K, V))
    out = torch.zeros((1, nq, H, 128), dtype=torch.bfloat16, device="cuda")
    dense_causal_attention(Qs, Ks, Vs, out=out.permute(0, 2, 1, 3))
    assert torch.equal(out.permute(0, 2, 1, 3), base)


def test_hook_routes_the_tail_through_the_kernel(lib, monkeypatch):
    from anchor_attention_b200 import patch
    import torch.nn.functional as F
    called = []
    real = F.scaled_dot_product_attention
    monkeypatch.setattr(F, "scaled_dot_product_attention", lambda *a, **k: called.append(1) or real(*a, **k))
    Q, K, V = (t.cuda() for t in make_inputs(2048, 2, 1, seed=9, rope=True))
    out = patch._dense_causal(Q[:, :, -500:], K, V, 128 ** -0.5, 2048 - 500)
    assert not called and out.shape == (1, 2, 500, 128)
    patch._dense_causal(Q[:, :, -1:], K, V, 128 ** -0.5, 2047)          # decode stays with the library
    assert called
