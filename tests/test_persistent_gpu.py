"""What the persistent form of steps 1 and 3 adds to the attention kernels: work items handed out by
a counter in the workspace, CTAs that see several items (or none), lists of very different lengths
inside one launch, and state that must not leak from one item, or one call, into the next.
Everything goes through the C ABI on a B200 and is compared with the CPU oracle or bit for bit with
another call."""
import pytest
import torch

from oracle.anchor_oracle import make_inputs, oracle_big_blocks
from parity_util import OUT_MAX_ABS, OUT_MEAN_ABS

pytestmark = pytest.mark.gpu


def _call(Q, K, V, theta, **kw):
    from anchor_attention_b200 import AnchorAttnCall
    return AnchorAttnCall(Q.cuda(), K.cuda(), V.cuda(), None, 128, 16, theta, **kw)


def _status_words(call):
    return call._view(call.layout.status_off, 4, torch.int32).cpu().tolist()


def test_every_item_is_handed_out_once_per_launch(lib):
    """Status word 3 counts the draws of the last step-1 / step-3 launch: every item once, plus one
    draw per CTA that found the counter exhausted.  Fewer items than SMs (some CTAs get nothing)
    and many more items than SMs."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for N, H, Hkv in ((2048, 2, 1), (16384, 8, 2)):
        Q, K, V = make_inputs(N, H, Hkv, seed=3, rope=True, q_shift=0.5)
        call = _call(Q, K, V, 9.0)
        items = H * N // 256
        ctas = min(items, sms)
        call.step1()
        torch.cuda.synchronize()
        assert _status_words(call)[3] == items + ctas
        call.step2()
        call.step3()
        torch.cuda.synchronize()
        st = _status_words(call)
        assert st[0] == 0 and st[3] == items + ctas
        call.check_status()


def test_repeated_calls_on_one_workspace_are_bit_identical(lib):
    """The counters are cleared by the entry points themselves: step 3 three times in a row, and a
    whole second forward, give the same bits (item-to-CTA assignment differs from run to run)."""
    Q, K, V = make_inputs(12288, 4, 2, seed=11, rope=True, q_shift=0.5)
    call = _call(Q, K, V, 10.0)
    first = call.run().clone()
    call.check_status()
    for _ in range(3):
        call.out.zero_()
        call.step3()
        assert torch.equal(call.out, first)
    call.out.zero_()
    assert torch.equal(call.run(), first)
    call.check_status()


@pytest.mark.parametrize("theta,q_shift,seed", [(8.0, 0.5, 5), (9.5, 0.5, 6), (12.0, 0.0, 7)])
def test_mixed_list_lengths_against_the_oracle(lib, theta, q_shift, seed):
    """One launch whose items range from empty lists (first big block, low theta) to lists of more
    than a hundred tiles, so that a CTA meets short and long items in turn: sampled big blocks of
    the first, a middle and the last query head against the oracle, and no NaN anywhere."""
    N, H, Hkv = 20480, 6, 2
    Q, K, V = make_inputs(N, H, Hkv, seed=seed, rope=True, q_shift=q_shift)
    call = _call(Q, K, V, theta)
    out = call.run().float().cpu()
    call.check_status()
    assert not torch.isnan(out).any()
    counts = call.counts.cpu()
    for h in (0, 3, 5):
        blocks = [0, 1, 5, 9]
        _, _, _, oids, oout = oracle_big_blocks(Q[0, h], K[0, h // (H // Hkv)], V[0, h // (H // Hkv)], blocks,
                                                None, 128, 16, theta)
        for b in blocks:
            rows = slice(b * 2048, (b + 1) * 2048)
            err = (out[0, h, rows] - oout[rows]).abs()
            assert err.max() <= OUT_MAX_ABS and err.mean() <= OUT_MEAN_ABS, (h, b, float(err.max()))
            assert abs(int(counts[0, h, b]) - oids[b].numel()) <= max(2, oids[b].numel() // 500)


def test_token_sharded_push_from_persistent_items(lib):
    """rows_per_peer > 0: every 128-row tile goes to the buffer of the rank that owns its tokens, at
    the row inside that rank's share -- also for items whose list is empty, which take their
    accumulator from the ring.  Both 'peers' are local buffers here."""
    N, H, Hkv, theta = 8192, 4, 2, 9.0
    Q, K, V = make_inputs(N, H, Hkv, seed=21, rope=True, q_shift=0.5)
    call = _call(Q, K, V, theta)
    want = call.run().clone()                                       # [1, H, N, D]
    call.check_status()
    half = N // 2
    shares = torch.zeros((2, 1, H, half, 128), dtype=torch.bfloat16, device="cuda")
    call2 = _call(Q, K, V, theta, out=shares[0])                    # strides of one share: [1, H, N/2, D]
    call2.step1()
    call2.step2()
    call2.step3_push([shares[0].data_ptr(), shares[1].data_ptr()], rows_per_peer=half)
    call2.check_status()
    assert torch.equal(shares[0], want[:, :, :half])
    assert torch.equal(shares[1], want[:, :, half:])


def test_two_streams_at_once(lib):
    """Two operator calls in flight on two streams, each with its own workspace: both grids are one
    CTA per SM and each SM holds one such CTA, so the second kernel's CTAs start as the first one's
    leave; nothing waits on another CTA, and both results equal the calls made one after the other."""
    probs = [(12288, 4, 2, 10.0, 31), (8192, 8, 2, 9.0, 32)]
    inputs = [tuple(t.cuda() for t in make_inputs(N, H, Hkv, seed=seed, rope=True, q_shift=0.5))
              for N, H, Hkv, _, seed in probs]
    from anchor_attention_b200 import AnchorAttnCall
    want = [AnchorAttnCall(*inp, None, 128, 16, p[3]).run().clone() for inp, p in zip(inputs, probs)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    calls = []
    for s, inp, p in zip(streams, inputs, probs):
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            calls.append(AnchorAttnCall(*inp, None, 128, 16, p[3]))
    for rep in range(3):                       # interleave the launches of the two calls
        for s, c in zip(streams, calls):
            with torch.cuda.stream(s):
                c.step1()
        for s, c in zip(streams, calls):
            with torch.cuda.stream(s):
                c.step2()
                c.step3()
    torch.cuda.synchronize()
    for c, w in zip(calls, want):
        c.check_status()
        assert torch.equal(c.out, w)


def test_step3_goes_kv_head_by_kv_head_when_the_lists_outgrow_the_scratch(lib):
    """A gather scratch too small for every tile any list could have: the plan kernel looks at the
    counts.  Lists that need more slots than there are -> step 3 runs KV head by KV head with the
    scratch reused (status word 4 = 1); lists that fit, or full lists (all runs) -> one go (0).
    Same bits as with the recommended workspace in every case."""
    from anchor_attention_b200 import AnchorAttnCall
    N, H, Hkv = 8192, 8, 4
    for theta, shift, slots, want_plan in ((10.0, 0.5, 40, 1),      # hundreds of gathered tiles, 40 slots
                                           (12.0, 0.0, 40, 0),      # full lists: no slot needed
                                           (8.5, 0.5, 400, 0)):     # short lists: a few dozen tiles fit
        Q, K, V = (t.cuda() for t in make_inputs(N, H, Hkv, seed=77, rope=True, q_shift=shift))
        ref_call = AnchorAttnCall(Q, K, V, None, 128, 16, theta)
        want = ref_call.run().clone()
        ref_call.check_status()
        need = int(sum((int(c) + 127) // 128 for b, row in enumerate(ref_call.counts[0].t().tolist()) for c in row
                       if c < max(b * 2048 - 256, 0)))
        probe = AnchorAttnCall(Q, K, V, None, 128, 16, theta)
        nbytes = probe.layout.min_bytes + slots * 65536
        call = AnchorAttnCall(Q, K, V, None, 128, 16, theta,
                              workspace=torch.empty(nbytes, dtype=torch.uint8, device="cuda"))
        out = call.run()
        call.check_status()
        st = _status_words_n(call, 5)
        assert st[4] == want_plan, (theta, need, slots, st)
        assert (need > slots) == bool(want_plan), (theta, need, slots)
        assert torch.equal(out, want)


def _status_words_n(call, n):
    return call._view(call.layout.status_off, n, torch.int32).cpu().tolist()
