"""Step 3's gather pass and the list validator, through the C ABI, on a B200.

The gather pass copies the K/V rows of id tiles that are not runs into scratch once;
the attention kernel then bulk-loads those tiles.  With no scratch, or too little, the
kernel gathers the remaining tiles itself.  All three routes must give the same bits."""
import ctypes

import pytest
import torch

from oracle.anchor_oracle import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,H,Hkv,theta,shift,block", [
    (8192, 4, 2, 10.0, 0.5, 128),      # sparse lists, hardly any run of 128 ids
    (8192, 2, 1, 11.0, 0.5, 128),      # dense lists with holes: runs and gathered tiles mixed
    (6144, 7, 1, 9.0, 0.5, 128),       # a few ids per list: partial last tiles only
    (8192, 2, 1, 10.0, 0.5, 256),      # other pooling block: other list capacities
])
def test_scratch_sizes_give_identical_bits(lib, N, H, Hkv, theta, shift, block):
    from anchor_attention_b200 import AnchorAttnCall
    Q, K, V = (t.cuda() for t in make_inputs(N, H, Hkv, seed=90, rope=True, q_shift=shift))
    outs, used = [], []
    for scratch in (0, None, 3 * 65536):
        ws = None
        call = AnchorAttnCall(Q, K, V, None, block, 16, theta, workspace=ws, gather_scratch_bytes=scratch)
        # a workspace of exactly the requested size (the cached one may be larger from earlier calls)
        nbytes = call.layout.total_bytes if scratch is None else call.layout.min_bytes + scratch
        call = AnchorAttnCall(Q, K, V, None, block, 16, theta,
                              workspace=torch.empty(nbytes, dtype=torch.uint8, device="cuda"))
        outs.append(call.run().clone())
        call.check_status()
        used.append(call.gather_slots_used if scratch != 0 else 0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert used[1] > 0, "the case is meant to have gathered tiles"
    assert used[2] >= min(used[1], 3)          # the counter runs past the capacity; three slots were filled
    print(f"\nN={N} H={H}: {used[1]} gathered tiles")


def test_validator_flags_bad_lists_without_gathering(lib):
    """A corrupted count and a corrupted id are each reported by the validator, which only
    reads the lists; no attention or gather kernel is launched on the corrupted workspace."""
    from anchor_attention_b200 import AnchorAttnCall
    Q, K, V = (t.cuda() for t in make_inputs(6144, 2, 1, seed=91, rope=True, q_shift=0.5))
    call = AnchorAttnCall(Q, K, V, None, 128, 16, 10.0)
    want = call.run().clone()
    call.validate_lists()
    call.check_status()                               # well formed
    counts, ids = call.counts, call.ids
    torch.cuda.synchronize()
    keep = int(counts[0, 1, 2])
    counts[0, 1, 2] = 2 * 2048 - 256 + 1              # one more than the list can hold
    call.validate_lists()
    with pytest.raises(RuntimeError, match="malformed"):
        call.check_status()
    counts[0, 1, 2] = keep
    off = call.id_row_offset(2)
    assert keep >= 2
    keep_id = int(ids[0, 1, off + 1])
    ids[0, 1, off + 1] = 6144 * 4                     # far outside the tensor
    call.validate_lists()
    with pytest.raises(RuntimeError, match="malformed"):
        call.check_status()
    ids[0, 1, off + 1] = int(ids[0, 1, off])          # inside the range but not ascending
    call.validate_lists()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.aa_check_status(ctypes.byref(call.params), stream) == -14
    ids[0, 1, off + 1] = keep_id
    call.validate_lists()
    call.check_status()
    assert torch.equal(call.step3(), want)
