"""The allocation-free stripe-identification entry point, through the C ABI.

Hosts such as an inference-runtime plug-in (whose enqueue hook may not allocate)
or a process whose device memory is fully owned by a framework arena cannot give
the library a freshly allocated workspace.  ``aa_step2_stripes_static`` serves
them from a fixed array inside the library; this test checks that it returns
exactly what the workspace-based ``aa_step2_stripes`` returns, on consecutive
calls that reuse (and so overwrite) that array, and that it refuses problems
the array cannot hold.

Collected last on purpose (file name), independent of every other test."""
import ctypes

import pytest
import torch

from oracle.anchor_oracle import make_inputs

pytestmark = pytest.mark.gpu


def _reference_lists(Q, K, V, theta):
    """counts, ids and the step-1 row maxima from the workspace-based entry points."""
    from anchor_attention_b200 import AnchorAttnCall
    call = AnchorAttnCall(Q, K, V, None, 128, 16, theta, workspace=None)
    call.step1()
    call.step2()
    torch.cuda.synchronize()
    return call.counts.clone(), call.ids.clone(), call.M.clone(), call.layout.ids_per_head


def _static_call(lib, Q, K, anchors, counts, ids, theta):
    from anchor_attention_b200 import _lib
    a = _lib.AAStripesStaticArgs()
    B, H, N, D = Q.shape
    a.B, a.H, a.Hkv, a.N, a.D = B, H, K.shape[1], N, D
    a.block_size, a.step, a.dtype = 128, 16, _lib.AA_BF16
    a.theta, a.sm_scale = theta, 0.0
    a.q, a.k = Q.data_ptr(), K.data_ptr()
    a.q_stride_b, a.q_stride_h, a.q_stride_n = Q.stride()[:3]
    a.k_stride_b, a.k_stride_h, a.k_stride_n = K.stride()[:3]
    a.anchors, a.counts, a.ids = anchors.data_ptr(), counts.data_ptr(), ids.data_ptr()
    return lib.aa_step2_stripes_static(ctypes.byref(a), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_entry_matches_workspace_entry_on_consecutive_calls(lib):
    problems = [(8192, 4, 2, 11.0, 0.5, 1), (4096, 2, 1, 12.0, 0.0, 0), (8192, 4, 2, 11.0, 0.5, 1)]
    prepared = []
    for N, H, Hkv, theta, shift, seed in problems:
        Q, K, V = (t.cuda() for t in make_inputs(N, H, Hkv, seed=seed, rope=True, q_shift=shift))
        counts_ref, ids_ref, M, ids_per_head = _reference_lists(Q, K, V, theta)
        # the caller owns the outputs; poison them so that stale values cannot pass
        counts = torch.full_like(counts_ref, -7)
        ids = torch.full((1, H, ids_per_head), -7, dtype=torch.int32, device="cuda")
        prepared.append((Q, K, M, counts, ids, theta, counts_ref, ids_ref))
    torch.cuda.synchronize()
    # back-to-back calls on one stream: each overwrites the shared array of the previous one
    for Q, K, M, counts, ids, theta, _, _ in prepared:
        assert _static_call(lib, Q, K, M, counts, ids, theta) == 0
    torch.cuda.synchronize()
    # none of the bounded device-side waits of these calls gave up (the word lives in the fixed array)
    assert lib.aa_step2_stripes_static_check_status(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    for Q, K, M, counts, ids, theta, counts_ref, ids_ref in prepared:
        assert torch.equal(counts, counts_ref)          # integer work: bit-exact
        assert int(counts.sum()) > 0 or theta < 5
        H, NB = counts.shape[1], counts.shape[2]
        from anchor_attention_b200 import _lib
        for h in range(H):
            for b in range(NB):
                off = _lib.load().aa_id_row_offset(128, 16, b)
                c = int(counts[0, h, b])
                assert torch.equal(ids[0, h, off:off + c], ids_ref[0, h, off:off + c])


def test_static_entry_refuses_what_does_not_fit(lib):
    from anchor_attention_b200 import _lib
    a = _lib.AAStripesStaticArgs()
    a.B, a.H, a.Hkv, a.N, a.D = 1, 32, 8, 131072, 128        # needs ~42 MB of intermediates
    a.block_size, a.step, a.dtype = 128, 16, _lib.AA_BF16
    a.theta = 12.0
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    a.q = a.k = a.anchors = a.counts = a.ids = dummy.data_ptr()
    a.q_stride_b = a.q_stride_h = a.q_stride_n = a.k_stride_b = a.k_stride_h = a.k_stride_n = 128
    rc = lib.aa_step2_stripes_static(ctypes.byref(a), None)
    assert rc == -12 and b"too large" in lib.aa_strerror(rc)
    a.step = 8
    assert lib.aa_step2_stripes_static(ctypes.byref(a), None) == -4
