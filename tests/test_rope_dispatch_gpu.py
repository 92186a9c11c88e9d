"""The fused rotary embedding + tokens->heads dispatch kernel on one GPU: both "peers" are local
buffers.  Must reproduce, bit for bit, what the library rotary function followed by a packing
copy gives (the arithmetic is bf16 products and sums, each rounded once, on both sides)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, qp, kp, vp, cos, sin, dst, H, Hkv, token0):
    from anchor_attention_b200 import _lib
    r = _lib.AARopeDispatch()
    n = qp.shape[0]
    r.n, r.H, r.Hkv, r.D, r.dtype = n, H, Hkv, 128, _lib.AA_BF16
    r.n_peers, r.token0 = len(dst), token0
    r.q, r.k, r.v = qp.data_ptr(), kp.data_ptr(), vp.data_ptr()
    r.q_stride_n, r.k_stride_n, r.v_stride_n = qp.stride(0), kp.stride(0), vp.stride(0)
    r.cos, r.sin = cos.data_ptr(), sin.data_ptr()
    for i, d in enumerate(dst):
        r.dst[i] = d.data_ptr()
    return lib.aa_rope_dispatch(ctypes.byref(r), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("n,H,Hkv,W,token0", [(300, 8, 4, 2, 512), (1024, 4, 2, 1, 0), (77, 8, 8, 4, 1000)])
def test_matches_library_rotary_and_packing(lib, n, H, Hkv, W, token0):
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    torch.manual_seed(n)
    D = 128
    N = token0 + n + 5
    # projection outputs as slices of one fused buffer (row stride larger than the row)
    fused = torch.randn(n, (H + 2 * Hkv) * D + 64, device="cuda").to(torch.bfloat16)
    qp, kp, vp = fused[:, :H * D], fused[:, H * D:(H + Hkv) * D], fused[:, (H + Hkv) * D:(H + 2 * Hkv) * D]
    pos = torch.arange(token0, token0 + n, device="cuda", dtype=torch.float32)
    inv = 500000.0 ** (-torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D)
    ang = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
    cos, sin = ang.cos().to(torch.bfloat16).contiguous(), ang.sin().to(torch.bfloat16).contiguous()
    h, hkv = H // W, Hkv // W
    dst = [torch.full((N, h + 2 * hkv, D), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    assert _call(lib, qp, kp, vp, cos, sin, dst, H, Hkv, token0) == 0
    torch.cuda.synchronize()
    q = qp.reshape(1, n, H, D).transpose(1, 2)
    k = kp.reshape(1, n, Hkv, D).transpose(1, 2)
    qr, kr = apply_rotary_pos_emb(q, k, cos[None], sin[None])
    qr, kr = qr.transpose(1, 2)[0], kr.transpose(1, 2)[0]              # [n, H, D]
    v = vp.reshape(n, Hkv, D)
    for d in range(W):
        rows = dst[d][token0:token0 + n]
        assert torch.equal(rows[:, :h], qr[:, d * h:(d + 1) * h])
        assert torch.equal(rows[:, h:h + hkv], kr[:, d * hkv:(d + 1) * hkv])
        assert torch.equal(rows[:, h + hkv:], v[:, d * hkv:(d + 1) * hkv])
        # nothing outside this rank's token rows was touched
        assert (dst[d][:token0] == 7.0).all() and (dst[d][token0 + n:] == 7.0).all()


def test_argument_checks(lib):
    from anchor_attention_b200 import _lib
    r = _lib.AARopeDispatch()
    assert lib.aa_rope_dispatch(None, None) == -1
    r.n, r.H, r.Hkv, r.D, r.n_peers = 16, 8, 4, 128, 3                 # 3 ranks do not divide the heads
    assert lib.aa_rope_dispatch(ctypes.byref(r), None) == -2
    r.n_peers, r.D = 2, 64
    assert lib.aa_rope_dispatch(ctypes.byref(r), None) == -3
    r.D = 128
    assert lib.aa_rope_dispatch(ctypes.byref(r), None) == -1           # NULL tensors
