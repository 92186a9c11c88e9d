"""Head-parallel host logic on CPU ranks (gloo, world size 2): the partition by KV
group and the single all-gather that assembles [B,N,H,D]."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from anchor_attention_b200.parallel import gather_heads, head_partition


def test_partition_covers_heads_in_kv_groups():
    for H, Hkv in ((32, 8), (28, 4), (8, 8)):
        for W in (1, 2, 4, 8):
            if Hkv % W:
                with pytest.raises(ValueError):
                    head_partition(H, Hkv, W, 0)
                continue
            seen_q, seen_kv = [], []
            for r in range(W):
                q_lo, q_hi, kv_lo, kv_hi = head_partition(H, Hkv, W, r)
                seen_q += list(range(q_lo, q_hi))
                seen_kv += list(range(kv_lo, kv_hi))
                g = H // Hkv
                assert all(h // g in range(kv_lo, kv_hi) for h in range(q_lo, q_hi))
            assert seen_q == list(range(H)) and seen_kv == list(range(Hkv))


def test_partition_rejects_bad_rank():
    with pytest.raises(ValueError):
        head_partition(32, 8, 2, 2)
    with pytest.raises(ValueError):
        head_partition(30, 8, 2, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, N, H, Hkv, D = 1, 64, 8, 4, 16
        full = torch.arange(B * N * H * D, dtype=torch.float32).view(B, N, H, D).to(torch.bfloat16)
        q_lo, q_hi, _, _ = head_partition(H, Hkv, world, rank)
        local = full[:, :, q_lo:q_hi].contiguous()
        got = gather_heads(local)
        ret[rank] = bool(torch.equal(got, full))
    finally:
        dist.destroy_process_group()


def test_gather_heads_two_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _worker_missing_peer(rank, world, port, ret):
    """Rank 1 leaves between steps (before the exchange); rank 0 must get an error from its
    collective within the short process-group timeout instead of waiting for ever."""
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    local = torch.zeros(1, 16, 2, 16, dtype=torch.bfloat16)
    gather_heads(local)                         # step 1: everybody takes part
    if rank == 1:
        ret[rank] = "left"
        return                                  # leaves with nothing in flight
    try:
        gather_heads(local)                     # step 2: the peer never joins
        ret[rank] = "no error"
    except Exception as e:                      # noqa: BLE001 - any failure report is what we want
        ret[rank] = "error: " + type(e).__name__


def test_missing_rank_is_reported_not_waited_for():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        ctx = mp.spawn(_worker_missing_peer, args=(world, port, ret), nprocs=world, join=False)
        for p in ctx.processes:
            p.join(timeout=60)
        alive = [p for p in ctx.processes if p.is_alive()]
        for p in alive:
            p.terminate()
        assert not alive, "a rank was still waiting for its missing peer after 60 s"
        assert ret.get(1) == "left"
        assert str(ret.get(0, "")).startswith("error"), dict(ret)
