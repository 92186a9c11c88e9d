"""Head-parallel execution on two GPUs (skipped on a single-GPU machine): the pushed
output, the all-gathered output and the single-GPU operator agree bit for bit."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, results):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        from anchor_attention_b200 import anchor_attn
        from anchor_attention_b200.parallel import HeadShardedAnchorAttn, head_partition
        from oracle.anchor_oracle import make_inputs
        N, H, Hkv, theta = 6144, 8, 4, 10.0
        Q, K, V = (t.cuda() for t in make_inputs(N, H, Hkv, seed=31, rope=True, q_shift=0.5))
        q_lo, q_hi, kv_lo, kv_hi = head_partition(H, Hkv, world, rank)
        want = anchor_attn(Q, K, V, difference=theta, return_computational_ratio=False).transpose(1, 2)
        ok = True
        for exchange in ("all_gather", "push"):
            op = HeadShardedAnchorAttn(difference=theta, exchange=exchange)
            for _ in range(3):          # three calls: the pushed output alternates between two copies
                got = op(Q[:, q_lo:q_hi], K[:, kv_lo:kv_hi], V[:, kv_lo:kv_hi])
            torch.cuda.synchronize()
            op.check_status()
            ok = ok and got.shape == (1, N, H, 128) and torch.equal(got, want)
            # the streamed host-buffer path: same assembled output on the device, this rank's
            # heads back in host memory
            hq, hk, hv = (t.cpu().pin_memory() for t in (Q[:, q_lo:q_hi], K[:, kv_lo:kv_hi], V[:, kv_lo:kv_hi]))
            hout = torch.empty((1, q_hi - q_lo, N, 128), dtype=torch.bfloat16).pin_memory()
            for _ in range(2):
                full = op.host_call(hq, hk, hv, hout)
            op.check_status()
            ok = ok and torch.equal(full, want) and torch.equal(hout.cuda().transpose(1, 2), want[:, :, q_lo:q_hi])
        results[rank] = bool(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_push_and_all_gather_match_single_gpu():
    import torch.multiprocessing as mp
    from anchor_attention_b200 import _lib
    _lib.load()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert results.get(0) is True and results.get(1) is True
