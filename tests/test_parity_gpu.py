"""CUDA path against the CPU oracle, through the C ABI, on a B200.

Tolerances.  Index sets: equal to the oracle's up to the documented tie band
(parity_util.tie_band).  Row maxima M: 2e-3 absolute (fp32 accumulation order
of a 128-term bf16 dot).  L: 2e-3 relative.  Acc: 1e-2 of the row's largest
entry, and 1e-2 absolute after normalising by L.  Output: max abs <= 2e-2 and mean abs <= 1e-3 (the north-star
tolerance against the reference's own output)."""
import pytest
import torch

from oracle.anchor_oracle import (anchor_attn_oracle, make_inputs, oracle_big_blocks, step2, step3)
from parity_util import OUT_MAX_ABS, OUT_MEAN_ABS, check_id_set

pytestmark = pytest.mark.gpu

SM = 128 ** -0.5


def _call(Q, K, V, theta, step=16):
    from anchor_attention_b200 import AnchorAttnCall
    return AnchorAttnCall(Q.cuda(), K.cuda(), V.cuda(), None, 128, step, theta)


CASES = [
    # N, H, Hkv, theta, rope, q_shift, seed
    (2048, 2, 1, 12.0, True, 0.0, 0),          # single big block: no stripes at all
    (4096, 4, 1, 12.0, True, 0.0, 0),          # headline distribution, density 1
    (8192, 4, 2, 11.0, False, 0.5, 1),         # sparse regime, two KV heads
    (8192, 7, 1, 9.0, True, 0.5, 2),           # Qwen-like group of 7, sparse with RoPE
    (6144, 2, 1, 10.0, True, 0.5, 2),          # same inputs as a golden fixture
    (8192, 2, 2, 4.0, False, 0.0, 3),          # theta small: (almost) nothing selected
]


@pytest.mark.parametrize("N,H,Hkv,theta,rope,q_shift,seed", CASES)
def test_full_operator_matches_oracle(lib, N, H, Hkv, theta, rope, q_shift, seed):
    Q, K, V = make_inputs(N, H, Hkv, seed=seed, rope=rope, q_shift=q_shift)
    ref = anchor_attn_oracle(Q, K, V, difference=theta, mode="bf16", order="tree")
    call = _call(Q, K, V, theta)
    call.step1()
    M, L, Acc = call.M.cpu(), call.L.cpu(), call.Acc.cpu()
    assert (M - ref.M).abs().max() < 2e-3
    assert ((L - ref.L).abs() / ref.L).max() < 2e-3
    # Acc is un-normalised: compare it relative to each row's own magnitude, and the
    # normalised step-1 output Acc / L absolutely
    scale = ref.Acc.abs().amax(dim=-1, keepdim=True).clamp_min(1.0)
    assert ((Acc - ref.Acc).abs() / scale).max() < 1e-2     # both sides round P to bf16 (2^-9 each)
    assert (Acc / L[..., None] - ref.Acc / ref.L[..., None]).abs().max() < 1e-2
    call.step2()
    ours = call.id_lists()
    counts = call.counts.cpu()
    g = H // Hkv
    total_band = total_diff = 0
    for h in range(H):
        for b in range(N // 2048):
            ids = ours[0][h][b]
            assert ids.numel() == counts[0, h, b]
            if b == 0:
                assert ids.numel() == 0
                continue
            assert (ids[1:] > ids[:-1]).all()
            if ids.numel():
                assert ids.min() >= 128 and ids.max() < b * 2048 - 128
            band, _ = check_id_set(ids, Q[0, h], K[0, h // g], ref.M[0, h], SM, theta, b)
            total_band += band
            total_diff += len(set(ids.tolist()) ^ set(ref.ids[0][h][b].tolist()))
    print(f"\nN={N} H={H}: selected {int(counts.sum())}, symmetric difference to oracle {total_diff}, "
          f"tie band {total_band}")
    call.step3()
    out = call.out.float().cpu()
    err = (out - ref.out).abs()
    assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS
    # the one-call entry point gives the same bits as the three steps
    from anchor_attention_b200 import anchor_attn
    out2, ratio = anchor_attn(Q.cuda(), K.cuda(), V.cuda(), difference=theta)
    assert torch.equal(out2.cpu(), call.out.cpu())
    assert abs(float(ratio) - float(counts.sum()) / ((H * N * N / 2048) // 2)) < 1e-6


GOLDEN_GPU = sorted(__import__("glob").glob(
    __import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "ref_gpu_bf16_*.npz")))


@pytest.mark.parametrize("path", GOLDEN_GPU, ids=[__import__("os").path.basename(p) for p in GOLDEN_GPU])
def test_against_reference_gpu_fixtures(lib, path):
    """Our kernels against what the reference's own compiled kernels produced on
    a B200 (bf16): state of step 1, index sets up to the tie band, final output
    within the north-star tolerance."""
    import numpy as np
    g = np.load(path)
    N, H, Hkv, theta = int(g["N"]), int(g["H"]), int(g["Hkv"]), float(g["theta"])
    block = int(g["block"]) if "block" in g.files else 128
    Q, K, V = make_inputs(N, H, Hkv, seed=int(g["seed"]), rope=bool(g["rope"]), q_shift=float(g["q_shift"]))
    from anchor_attention_b200 import AnchorAttnCall
    call = AnchorAttnCall(Q.cuda(), K.cuda(), V.cuda(), None, block, 16, theta)
    out = call.run().float().cpu()
    call.check_status()
    assert (call.M.cpu()[0] - torch.from_numpy(g["M"])).abs().max() < 1e-4
    assert ((call.L.cpu()[0] - torch.from_numpy(g["L"])).abs() / torch.from_numpy(g["L"])).max() < 1e-4
    acc, acc_ref = call.Acc.cpu()[0, :, ::16], torch.from_numpy(g["Acc_rows16"])
    row_scale = acc_ref.abs().amax(dim=-1, keepdim=True).clamp_min(1.0)
    assert ((acc - acc_ref).abs() / row_scale).max() < 1e-2     # both sides round P to bf16 (2^-9 each)
    ours = call.id_lists()
    pos = diff = total = band = 0
    Mref = torch.from_numpy(g["M"])
    for h in range(H):
        for b in range(N // (block * 16)):
            c = int(g["counts"][h, b])
            ref_ids = g["ids"][pos:pos + c]
            pos += c
            total += c
            if b:
                # both our set and the reference's own set obey the exact decision outside the tie band
                band += check_id_set(ours[0][h][b], Q[0, h], K[0, h // (H // Hkv)], Mref[h], SM, theta, b, block)[0]
                check_id_set(torch.from_numpy(ref_ids.astype("int64")), Q[0, h], K[0, h // (H // Hkv)], Mref[h], SM,
                             theta, b, block)
            diff += len(set(ref_ids.tolist()) ^ set(ours[0][h][b].tolist()))
    print(f"\n{__import__('os').path.basename(path)}: {total} selected by the reference, symmetric difference {diff}, "
          f"tie band {band}")
    assert diff <= band          # the two sets can only differ inside the band
    out_ref = torch.from_numpy(g["out"]).view(torch.bfloat16).float()
    err = (out[0] - out_ref).abs()
    assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS


def test_step3_given_oracle_state(lib):
    """Step 3 alone: our kernel fed with OUR ids and state equals the oracle's
    step 3 fed with the same ids and state (isolates the gathered attention)."""
    N, H = 8192, 2
    Q, K, V = make_inputs(N, H, 1, seed=4, rope=True, q_shift=0.5)
    call = _call(Q, K, V, 9.5)
    call.step1()
    call.step2()
    ids = call.id_lists()
    M, L, Acc = call.M.cpu(), call.L.cpu(), call.Acc.cpu()
    call.step3()
    out = call.out.float().cpu()
    for h in range(H):
        want = step3(Q[0, h], K[0, 0], V[0, 0], ids[0][h], M[0, h], L[0, h], Acc[0, h], SM)
        err = (out[0, h] - want).abs()
        assert err.max() <= OUT_MAX_ABS and err.mean() <= 2e-4     # max: one bf16 ulp of values in [2, 4)


def test_step32(lib):
    N, H = 8192, 2
    Q, K, V = make_inputs(N, H, 1, seed=6, rope=True, q_shift=0.5)
    ref = anchor_attn_oracle(Q, K, V, step=32, difference=9.5)
    call = _call(Q, K, V, 9.5, step=32)
    out = call.run().float().cpu()
    err = (out - ref.out).abs()
    assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS
    # index sets: equal to the exact decision outside the tie band, as for step 16
    ours = call.id_lists()
    band = diff = 0
    for h in range(H):
        for b in range(1, N // (128 * 32)):
            band += check_id_set(ours[0][h][b], Q[0, h], K[0, 0], ref.M[0, h], SM, 9.5, b, 128, 32)[0]
            diff += len(set(ours[0][h][b].tolist()) ^ set(ref.ids[0][h][b].tolist()))
    print(f"\nstep 32: selected {int(call.counts.sum())}, symmetric difference to oracle {diff}, tie band {band}")
    assert diff <= band


def test_strided_layouts_and_expanded_kv(lib):
    """[B,N,H,D] memory order (what the attention module holds) and K/V already
    expanded to H heads (what the reference's caller passes) give identical bits."""
    from anchor_attention_b200 import anchor_attn
    N, H, Hkv = 4096, 4, 2
    Q, K, V = make_inputs(N, H, Hkv, seed=8, rope=True, q_shift=0.5)
    Qc, Kc, Vc = Q.cuda(), K.cuda(), V.cuda()
    base = anchor_attn(Qc, Kc, Vc, difference=9.5, return_computational_ratio=False)
    Qs = Qc.transpose(1, 2).contiguous().transpose(1, 2)          # B,N,H,D memory
    Ks = Kc.transpose(1, 2).contiguous().transpose(1, 2)
    Vs = Vc.transpose(1, 2).contiguous().transpose(1, 2)
    assert not Qs.is_contiguous()
    assert torch.equal(anchor_attn(Qs, Ks, Vs, difference=9.5, return_computational_ratio=False), base)
    Ke, Ve = Kc.repeat_interleave(H // Hkv, dim=1), Vc.repeat_interleave(H // Hkv, dim=1)
    assert torch.equal(anchor_attn(Qc, Ke, Ve, difference=9.5, return_computational_ratio=False), base)


def test_timing_entry_point_mirrors_the_reference(lib):
    """anchor_attn_test_time: same output as anchor_attn, plus the two phase times."""
    from anchor_attention_b200 import anchor_attn, anchor_attn_test_time
    Q, K, V = (t.cuda() for t in make_inputs(4096, 2, 1, seed=3, rope=True, q_shift=0.5))
    out, ratio, search_ms, compute_ms = anchor_attn_test_time(Q, K, V, difference=10)
    want, want_ratio = anchor_attn(Q, K, V, difference=10)
    assert torch.equal(out, want) and float(ratio) == float(want_ratio)
    assert search_ms > 0 and compute_ms > 0
    out2, s2, c2 = anchor_attn_test_time(Q, K, V, difference=10, return_computational_ratio=False)
    assert torch.equal(out2, want)


def test_reference_layout_export(lib):
    N, H = 6144, 2
    Q, K, V = make_inputs(N, H, 1, seed=2, rope=True, q_shift=0.5)
    call = _call(Q, K, V, 10.0)
    call.step1()
    call.step2()
    coords, counts = call.coords_reference_layout()
    assert coords.shape == (1, H, 3, N) and counts.shape == (1, H, 3, 1)
    lists = call.id_lists()
    for h in range(H):
        for b in range(3):
            c = int(counts[0, h, b, 0])
            assert torch.equal(coords[0, h, b, :c].cpu(), lists[0][h][b])
    # the host-side sum of the counts (numerator of the reference's sparsity ratio)
    import ctypes
    total = ctypes.c_int64(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.aa_total_selected(ctypes.byref(call.params), stream, ctypes.byref(total)) == 0
    assert total.value == int(counts.sum())
    assert abs(float(call.ratio()) - total.value / ((H * N * N / 2048) // 2)) < 1e-6


def test_full_size_sampled_blocks_and_properties(lib):
    """BASELINE configs[1] shape (N=32768, 32/8 heads): checked through
    size-independent properties and the oracle on sampled (head, big block) pairs."""
    N, H, Hkv = 32768, 32, 8
    Q, K, V = make_inputs(N, H, Hkv, seed=0, rope=True)
    Qc, Kc, Vc = Q.cuda(), K.cuda(), V.cuda()
    from anchor_attention_b200 import AnchorAttnCall
    call = AnchorAttnCall(Qc, Kc, Vc, None, 128, 16, 12.0)
    out = call.run()
    counts = call.counts.cpu()
    ids = call.ids.cpu()
    # property: every list ascending, inside its candidate range
    for h in (0, 5, 31):
        for b in range(1, 16):
            c = int(counts[0, h, b])
            seg = ids[0, h, call.id_row_offset(b): call.id_row_offset(b) + c]
            assert c <= b * 2048 - 256 and (seg[1:] > seg[:-1]).all() and seg[0] >= 128 and seg[-1] < b * 2048 - 128
    # on this distribution theta = 12 selects every candidate
    assert int(counts.sum()) == 32 * sum(b * 2048 - 256 for b in range(1, 16))
    # property: the operator is linear in V (selection depends on Q and K only)
    V2 = torch.randn_like(V, dtype=torch.float32).to(torch.bfloat16).cuda()
    o1 = out.float()
    o2 = AnchorAttnCall(Qc, Kc, V2, None, 128, 16, 12.0, workspace=torch.empty_like(call.workspace)).run().float()
    o12 = AnchorAttnCall(Qc, Kc, (Vc.float() + V2.float()).to(torch.bfloat16), None, 128, 16, 12.0,
                         workspace=torch.empty_like(call.workspace)).run().float()
    # three bf16-rounded outputs and a bf16-rounded V sum: a few ulps of the operands
    assert ((o12 - (o1 + o2)).abs() / (1 + o1.abs() + o2.abs())).max() < 2e-2
    # oracle on sampled big blocks
    outc = out.float().cpu()
    for h, b in ((0, 0), (13, 7), (31, 15)):
        M, L, Acc, oids, oout = oracle_big_blocks(Q[0, h], K[0, h // 4], V[0, h // 4], [b])
        rows = slice(b * 2048, (b + 1) * 2048)
        err = (outc[0, h, rows] - oout[rows]).abs()
        assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS
        assert int(counts[0, h, b]) == oids[b].numel()


def test_step3_push_writes_every_copy(lib):
    """The push variant of step 3 (used head-parallel) stores the same bits as step 3 into
    each of the given output copies; here both copies are local buffers."""
    from anchor_attention_b200 import AnchorAttnCall
    Q, K, V = (t.cuda() for t in make_inputs(6144, 4, 2, seed=41, rope=True, q_shift=0.5))
    copies = torch.zeros((2, 1, 6144, 6, 128), dtype=torch.bfloat16, device="cuda")    # two [B,N,H+2,D] buffers
    view = copies[0][:, :, 1:5].permute(0, 2, 1, 3)                                    # heads 1..4 of copy 0
    call = AnchorAttnCall(Q, K, V, None, 128, 16, 10.0, out=view)
    call.step1()
    call.step2()
    head_off = 1 * 128 * 2
    call.step3_push([copies[0].data_ptr() + head_off, copies[1].data_ptr() + head_off])
    call.check_status()
    want = AnchorAttnCall(Q, K, V, None, 128, 16, 10.0).run().transpose(1, 2)
    for c in range(2):
        assert torch.equal(copies[c][:, :, 1:5], want)
        assert not copies[c][:, :, 0].any() and not copies[c][:, :, 5].any()


def test_batch_fused_qkv_and_padded_heads(lib):
    """Batch of two; Q/K/V as slices of one fused [B,N,(H+2*Hkv)*D] projection output; K/V
    heads separated by padding (no 2-D tensor map covers them, so the gathers fall back to
    cp.async only).  All give the bits of the plain contiguous call, batch by batch."""
    from anchor_attention_b200 import anchor_attn
    N, H, Hkv, theta = 6144, 4, 2, 10.0
    parts = [make_inputs(N, H, Hkv, seed=s, rope=True, q_shift=0.5) for s in (51, 52)]
    Q, K, V = (torch.cat([p[i] for p in parts], dim=0).cuda() for i in range(3))
    per_batch = [anchor_attn(*(t.cuda() for t in p), difference=theta, return_computational_ratio=False)
                 for p in parts]
    base = torch.cat(per_batch, dim=0)
    assert torch.equal(anchor_attn(Q, K, V, difference=theta, return_computational_ratio=False), base)
    # fused projection output, token-major: [B, N, (H + 2 Hkv) * D]
    fused = torch.cat([Q.transpose(1, 2).reshape(2, N, H * 128), K.transpose(1, 2).reshape(2, N, Hkv * 128),
                       V.transpose(1, 2).reshape(2, N, Hkv * 128)], dim=2).contiguous()
    Qf = fused[:, :, :H * 128].view(2, N, H, 128).transpose(1, 2)
    Kf = fused[:, :, H * 128:(H + Hkv) * 128].view(2, N, Hkv, 128).transpose(1, 2)
    Vf = fused[:, :, (H + Hkv) * 128:].view(2, N, Hkv, 128).transpose(1, 2)
    assert torch.equal(anchor_attn(Qf, Kf, Vf, difference=theta, return_computational_ratio=False), base)
    # heads padded apart by 8 elements: head stride N*128 + 8
    def padded(x):
        B, h, n, d = x.shape
        buf = torch.zeros((B, h, n * d + 8), dtype=x.dtype, device=x.device)
        buf[:, :, :n * d] = x.reshape(B, h, n * d)
        return buf[:, :, :n * d].view(B, h, n, d)
    Kp, Vp = padded(K), padded(V)
    assert Kp.stride(1) == N * 128 + 8
    assert torch.equal(anchor_attn(Q, Kp, Vp, difference=theta, return_computational_ratio=False), base)


def test_bounded_wait_reports_timeout_and_context_survives(lib):
    """A device-side wait that can never be satisfied gives up after its poll limit and sets
    the status word; the host reads AA_ERR_DEVICE_TIMEOUT, and the next operator call on the
    same context works (nothing trapped or faulted)."""
    import ctypes
    from anchor_attention_b200 import AnchorAttnCall, _lib
    Q, K, V = (t.cuda() for t in make_inputs(4096, 2, 1, seed=71, rope=True))
    call = AnchorAttnCall(Q, K, V, None, 128, 16, 12.0)
    want = call.run().clone()
    call.check_status()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.aa_selftest_wait_timeout(ctypes.byref(call.params), stream) == 0
    assert lib.aa_check_status(ctypes.byref(call.params), stream) == -11            # AA_ERR_DEVICE_TIMEOUT
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        call.check_status()
    got = call.run()                        # clears the status word again
    call.check_status()
    assert torch.equal(got, want)


@pytest.mark.parametrize("block,N,H,Hkv,theta", [(64, 4096, 4, 2, 10.0), (256, 8192, 2, 1, 10.0), (64, 2048, 2, 1, 12.0)])
def test_other_pooling_block_sizes(lib, block, N, H, Hkv, theta):
    """block_size 64 and 256 (big blocks of 1024 / 4096 rows, candidates [block, b*G - block)):
    state, index sets up to the tie band and output against the oracle."""
    from anchor_attention_b200 import AnchorAttnCall
    Q, K, V = make_inputs(N, H, Hkv, seed=80 + block, rope=True, q_shift=0.5)
    ref = anchor_attn_oracle(Q, K, V, block_size=block, difference=theta, mode="bf16", order="tree")
    call = AnchorAttnCall(Q.cuda(), K.cuda(), V.cuda(), None, block, 16, theta)
    out = call.run().float().cpu()
    call.check_status()
    assert (call.M.cpu() - ref.M).abs().max() < 2e-3
    assert ((call.L.cpu() - ref.L).abs() / ref.L).max() < 2e-3
    G = block * 16
    ours, counts = call.id_lists(), call.counts.cpu()
    total_diff = 0
    for h in range(H):
        for b in range(N // G):
            ids = ours[0][h][b]
            assert ids.numel() == counts[0, h, b]
            if b == 0:
                assert ids.numel() == 0
                continue
            assert (ids[1:] > ids[:-1]).all()
            if ids.numel():
                assert ids.min() >= block and ids.max() < b * G - block
            check_id_set(ids, Q[0, h], K[0, h // (H // Hkv)], ref.M[0, h], SM, theta, b, block)
            total_diff += len(set(ids.tolist()) ^ set(ref.ids[0][h][b].tolist()))
    print(f"\nblock {block}: selected {int(counts.sum())}, symmetric difference to oracle {total_diff}")
    assert int(counts.sum()) > 0
    err = (out - ref.out).abs()
    assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS
