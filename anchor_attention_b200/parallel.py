"""Head-parallel execution: the query heads are partitioned by KV-head group
across the ranks of one node and the head outputs are exchanged with a single
all-gather (NCCL on GPUs; gloo works for the host-side logic on CPU ranks).

The reference is single-GPU (test_hf.py:126 pins one device); every (batch,
query head) is independent through all three steps of the operator
(anchor_attn/src/ops/anchor_attn_v4.py:226-273), so this is the one natural
partition and the all-gather its only exchange."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def head_partition(H: int, Hkv: int, world_size: int, rank: int) -> Tuple[int, int, int, int]:
    """(q_lo, q_hi, kv_lo, kv_hi) owned by ``rank``: whole KV groups, in order."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if H % Hkv != 0:
        raise ValueError(f"{Hkv} KV heads do not divide {H} query heads")
    if Hkv % world_size != 0:
        raise ValueError(f"world size {world_size} does not divide the {Hkv} KV heads")
    per = Hkv // world_size
    g = H // Hkv
    return rank * per * g, (rank + 1) * per * g, rank * per, (rank + 1) * per


def gather_heads(local_out: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather of head outputs.  ``local_out`` is this rank's [B, N, h, D]
    block (token-major, so that the gathered result feeds the output projection);
    returns [B, N, W*h, D] on every rank.  One collective."""
    W = dist.get_world_size(group)
    B, N, h, D = local_out.shape
    if W == 1:
        return local_out
    if out is None:
        out = torch.empty((W, B, N, h, D), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(out.view(W * B, N, h, D), local_out.contiguous(), group=group)
    # [W,B,N,h,D] -> [B,N,W,h,D] -> [B,N,W*h,D]
    return out.permute(1, 2, 0, 3, 4).reshape(B, N, W * h, D)


class PushedOutput:
    """The assembled [B, N, H, D] output of a head-parallel layer, kept in symmetric
    memory (every rank can address every rank's copy) so that step 3 stores each of its
    rows into all copies while it computes; no all-gather follows, only a barrier.
    Two copies alternate from call to call: a rank may still be reading the previous
    layer's result while a faster peer already writes the next one."""

    def __init__(self, B, N, H, D, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        self.shape = (B, N, H, D)
        self.bufs = [symm_mem.empty((B, N, H, D), dtype=dtype, device=device) for _ in range(2)]
        self.handles = [symm_mem.rendezvous(b, group) for b in self.bufs]
        self.turn = 0

    def next(self):
        """(local tensor [B,N,H,D], every rank's base pointer of it, handle) for this call."""
        i = self.turn
        self.turn ^= 1
        h = self.handles[i]
        return self.bufs[i], [int(p) for p in h.buffer_ptrs], h


class HeadShardedAnchorAttn:
    """anchor_attn on this rank's heads followed by the all-gather.  Q [B,h,N,D],
    K/V [B,hkv,N,D] hold only the heads ``head_partition`` assigns to the rank."""

    def __init__(self, sm_scale=None, block_size=128, step=16, difference=12.0, group=None, exchange="all_gather"):
        """``exchange``: "all_gather" (one NCCL collective after the operator) or "push"
        (step 3 stores its rows into every rank's copy of the output over NVLink; a
        barrier instead of a collective)."""
        if exchange not in ("all_gather", "push"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.sm_scale, self.block_size, self.step, self.difference = sm_scale, block_size, step, difference
        self.group = group
        self.exchange = exchange
        self._local = None
        self._gathered = None
        self._pushed = None

    def _call_push(self, Q, K, V):
        from .ops import AnchorAttnCall
        B, h, N, D = Q.shape
        W, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        H = W * h
        if self._pushed is None or self._pushed.shape != (B, N, H, D):
            self._pushed = PushedOutput(B, N, H, D, Q.dtype, Q.device, self.group)
        buf, ptrs, handle = self._pushed.next()
        mine = buf[:, :, rank * h:(rank + 1) * h]                       # this rank's heads inside the copy
        call = AnchorAttnCall(Q, K, V, self.sm_scale, self.block_size, self.step, self.difference,
                              out=mine.permute(0, 2, 1, 3))
        call.step1()
        call.step2()
        head_off = rank * h * D * buf.element_size()
        call.step3_push([p + head_off for p in ptrs])
        handle.barrier(channel=0)
        self.last_call = call
        return buf

    def __call__(self, Q, K, V):
        from .ops import AnchorAttnCall
        if self.exchange == "push" and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            return self._call_push(Q, K, V)
        B, h, N, D = Q.shape
        if self._local is None or self._local.shape != (B, N, h, D):
            self._local = torch.empty((B, N, h, D), dtype=Q.dtype, device=Q.device)
            W = dist.get_world_size(self.group) if dist.is_initialized() else 1
            self._gathered = torch.empty((W, B, N, h, D), dtype=Q.dtype, device=Q.device) if W > 1 else None
        # the kernels write straight into token-major memory through the output strides
        call = AnchorAttnCall(Q, K, V, self.sm_scale, self.block_size, self.step, self.difference,
                              out=self._local.permute(0, 2, 1, 3))
        call.run()
        self.last_call = call
        if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return self._local
        return gather_heads(self._local, self.group, self._gathered)
