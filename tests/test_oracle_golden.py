"""The CPU oracle against golden vectors produced by the reference's own kernels
(tests/golden/make_golden.py: reference Triton kernels run by Triton's CPU
interpreter in fp16).  Index sets and row maxima must match exactly; the other
quantities to fp32/fp16 rounding."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle.anchor_oracle import (anchor_attn_oracle, make_inputs, step1, step2, step2_dense_check,
                                  dense_causal_attention)

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_interp_fp16_*.npz")))
GOLDEN_GPU = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_gpu_bf16_*.npz")))


def _block(g):
    """Pooling block size of a fixture (the first fixtures were written before the key existed)."""
    return int(g["block"]) if "block" in g.files else 128


def _inputs(g):
    return make_inputs(int(g["N"]), int(g["H"]), int(g["Hkv"]), seed=int(g["seed"]), rope=bool(g["rope"]),
                       dtype=torch.float16, q_shift=float(g["q_shift"]))


def test_golden_files_present():
    assert len(GOLDEN) >= 3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_kernels(path):
    g = np.load(path)
    Q, K, V = _inputs(g)
    # the interpreter sums the pooled queries left to right and adds diff in fp16
    r = anchor_attn_oracle(Q, K, V, block_size=_block(g), difference=float(g["theta"]), mode="fp16", order="seq",
                           diff_add="input")
    H = int(g["H"])
    assert r.counts[0].tolist() == g["counts"].tolist()
    flat = np.concatenate([x.numpy() for h in range(H) for x in r.ids[0][h]])
    assert flat.shape == g["ids"].shape and (flat == g["ids"]).all()          # bit-exact index sets
    assert np.array_equal(r.M[0].numpy(), g["M"])                               # row maxima exact
    assert np.max(np.abs(r.L[0].numpy() - g["L"]) / g["L"]) < 2e-6
    # fp32 accumulation-order noise grows with the window length (4096 keys at block 256)
    assert np.max(np.abs(r.Acc[0, :, ::16].numpy() - g["Acc_rows16"])) < 2e-5 * max(1, _block(g) // 128)
    out_ref = g["out"].astype(np.float32)
    err = np.abs(r.out[0].numpy() - out_ref)
    assert err.max() <= 2e-2 and err.mean() <= 1e-3
    assert abs(r.ratio - float(g["ratio"])) < 1e-6


@pytest.mark.parametrize("path", GOLDEN_GPU, ids=[os.path.basename(p) for p in GOLDEN_GPU])
def test_oracle_matches_reference_kernels_on_gpu_bf16(path):
    """Fixtures written by the reference's compiled Triton kernels on a B200 in
    bf16.  fp32 accumulation order differs between a CPU matmul and the tensor
    cores, so index sets are compared up to the tie band and M, L, Acc to
    accumulation-order noise."""
    from parity_util import check_id_set
    g = np.load(path)
    N, H, Hkv, theta = int(g["N"]), int(g["H"]), int(g["Hkv"]), float(g["theta"])
    Q, K, V = make_inputs(N, H, Hkv, seed=int(g["seed"]), rope=bool(g["rope"]), dtype=torch.bfloat16,
                          q_shift=float(g["q_shift"]))
    block = _block(g)
    r = anchor_attn_oracle(Q, K, V, block_size=block, difference=theta, mode="bf16", order="tree")
    assert np.abs(r.M[0].numpy() - g["M"]).max() < 1e-4
    assert (np.abs(r.L[0].numpy() - g["L"]) / g["L"]).max() < 1e-4
    assert np.abs(r.Acc[0, :, ::16].numpy() - g["Acc_rows16"]).max() < 5e-3
    pos, diff, total = 0, 0, 0
    for h in range(H):
        for b in range(N // (block * 16)):
            c = int(g["counts"][h, b])
            ref_ids = torch.from_numpy(g["ids"][pos:pos + c].astype(np.int32))
            pos += c
            total += c
            if b == 0:
                assert c == 0
                continue
            # the reference's own list must sit inside our tie band classification ...
            check_id_set(ref_ids, Q[0, h], K[0, h // (H // Hkv)], r.M[0, h], 128 ** -0.5, theta, b, block)
            diff += len(set(ref_ids.tolist()) ^ set(r.ids[0][h][b].tolist()))
    assert diff <= max(2, 0.01 * total), f"{diff} of {total} selected columns differ"
    out_ref = torch.from_numpy(g["out"]).view(torch.bfloat16).float()
    err = (r.out[0] - out_ref).abs()
    assert err.max() <= 2e-2 and err.mean() <= 1e-3


def test_ids_ascending_and_in_candidate_range():
    g = np.load(GOLDEN[-1])
    Q, K, V = _inputs(g)
    r = anchor_attn_oracle(Q, K, V, difference=float(g["theta"]), mode="fp16")
    for h in range(int(g["H"])):
        for b, ids in enumerate(r.ids[0][h]):
            if ids.numel():
                assert (ids[1:] > ids[:-1]).all()
                assert ids.min() >= 128 and ids.max() < b * 2048 - 128


def test_fp32_step2_equals_reference_dense_formulation():
    Q, K, V = make_inputs(6144, 1, 1, seed=3, rope=False, dtype=None, q_shift=0.5)
    M, L, Acc = step1(Q[0, 0], K[0, 0], V[0, 0], 128 ** -0.5, mode="fp32")
    a = step2(Q[0, 0], K[0, 0], M, 128 ** -0.5, 11.0, mode="fp32")
    b = step2_dense_check(Q[0, 0], K[0, 0], M, 128 ** -0.5, 11.0)
    assert [x.tolist() for x in a] == [x.tolist() for x in b]
    assert 0 < sum(x.numel() for x in a) < 1792 + 3840


def test_quirks_double_count_and_never_attended():
    """A selected column inside the first 2048 keys is used twice, and the 128 keys
    just before a big block (b >= 2) are never attended: with every candidate
    selected the result must differ from dense attention exactly as predicted."""
    N = 6144
    Q, K, V = make_inputs(N, 1, 1, seed=5, rope=False, dtype=None)
    r = anchor_attn_oracle(Q, K, V, difference=1e4, mode="fp32")       # theta huge: all candidates selected
    assert r.counts[0, 0].tolist() == [0, 1792, 3840]
    q, k, v = Q[0, 0], K[0, 0], V[0, 0]
    s = (q @ k.T) * (128 ** -0.5)
    row = 2 * 2048 + 77                                                 # a row of big block 2
    w = torch.zeros(N)
    w[:2048] += 1                                                       # init window
    w[4096:row + 1] += 1                                                # own big block, causal
    w[128:4096 - 128] += 1                                              # stripe candidates of big block 2
    p = torch.exp(s[row] - s[row].max()) * w
    expect = (p / p.sum()) @ v
    assert torch.allclose(r.out[0, 0, row], expect, atol=2e-5)
    assert w[4096 - 128:4096].sum() == 0 and w[128:2048].min() == 2


def test_rejects_bad_arguments():
    Q, K, V = make_inputs(2048, 1, 1, dtype=None)
    with pytest.raises(AssertionError):
        anchor_attn_oracle(Q, K, V, step=8)
    with pytest.raises(AssertionError):
        anchor_attn_oracle(Q[:, :, :1000], K[:, :, :1000], V[:, :, :1000])


def test_single_big_block_is_plain_causal_attention():
    Q, K, V = make_inputs(2048, 2, 1, seed=7, rope=True, dtype=None)
    r = anchor_attn_oracle(Q, K, V, mode="fp32")
    assert r.counts.sum() == 0
    d = dense_causal_attention(Q, K, V)
    assert torch.allclose(r.out, d, atol=1e-4)
