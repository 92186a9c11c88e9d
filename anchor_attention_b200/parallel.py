"""Head-parallel execution: the query heads are partitioned by KV-head group
across the ranks of one node.  The head outputs reach every rank either because
step 3 stores its rows into every rank's copy of the assembled output over NVLink
while it computes (a bounded flag barrier follows), or through a single all-gather
(NCCL on GPUs; gloo works for the host-side logic on CPU ranks).

The reference is single-GPU (test_hf.py:126 pins one device); every (batch,
query head) is independent through all three steps of the operator
(anchor_attn/src/ops/anchor_attn_v4.py:226-273), so this is the one natural
partition and the output exchange its only communication."""
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
    layer's result while a faster peer already writes the next one.

    The barrier is the library's own flag barrier (``aa_peer_barrier``: plain peer stores
    and loads on a small symmetric flag array, bounded wait).  If a peer never arrives it
    gives up after ``timeout_ms``, sets a status word and returns; ``check_status()``
    raises then.  Nothing on this path can spin for ever."""

    def __init__(self, B, N, H, D, dtype, device, group=None, timeout_ms: int = 10000):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _lib.MAX_PEERS:
            raise ValueError("at most 8 ranks (one node)")
        self.shape = (B, N, H, D)
        self.device = torch.device(device)
        self.bufs = [symm_mem.empty((B, N, H, D), dtype=dtype, device=device) for _ in range(2)]
        self.handles = [symm_mem.rendezvous(b, group) for b in self.bufs]
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flag_handle = symm_mem.rendezvous(self.flags, group)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)                  # every rank's flags are zero before anyone announces an epoch
        self.timeout_ms = int(timeout_ms)
        self.epoch = 0
        self.turn = 0
        self._lib = _lib

    def next(self):
        """(local tensor [B,N,H,D], every rank's base pointer of it) for this call."""
        i = self.turn
        self.turn ^= 1
        return self.bufs[i], [int(p) for p in self.handles[i].buffer_ptrs]

    def barrier(self):
        """Enqueue the flag barrier on the current stream (no host synchronisation)."""
        import ctypes
        self.epoch += 1
        b = self._lib.AAPeerBarrier()
        b.n_peers, b.rank, b.epoch, b.timeout_ms = self.world, self.rank, self.epoch, self.timeout_ms
        for i, ptr in enumerate(self.flag_handle.buffer_ptrs):
            b.flags[i] = int(ptr)
        b.status = self.status.data_ptr()
        with torch.cuda.device(self.device):
            rc = self._lib.load().aa_peer_barrier(ctypes.byref(b),
                                                  ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        if rc != self._lib.AA_OK:
            raise RuntimeError(f"aa_peer_barrier: {self._lib.error_text(rc)}")

    def check_status(self):
        """Synchronises; raises if a barrier of this object gave up waiting for a peer."""
        if int(self.status.item()) != 0:
            raise RuntimeError("head-parallel barrier: a peer did not arrive within "
                               f"{self.timeout_ms} ms; the assembled output is incomplete")


class HeadShardedAnchorAttn:
    """anchor_attn on this rank's heads followed by the exchange.  Q [B,h,N,D],
    K/V [B,hkv,N,D] hold only the heads ``head_partition`` assigns to the rank."""

    def __init__(self, sm_scale=None, block_size=128, step=16, difference=12.0, group=None, exchange="all_gather",
                 timeout_ms: int = 10000):
        """``exchange``: "all_gather" (one NCCL collective after the operator) or "push"
        (step 3 stores its rows into every rank's copy of the output over NVLink; a
        bounded flag barrier instead of a collective)."""
        if exchange not in ("all_gather", "push"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.sm_scale, self.block_size, self.step, self.difference = sm_scale, block_size, step, difference
        self.group = group
        self.exchange = exchange
        self.timeout_ms = timeout_ms
        self._local = None
        self._gathered = None
        self._pushed = None
        self._host = None

    def _pushed_output(self, B, N, H, D, dtype, device):
        if self._pushed is None or self._pushed.shape != (B, N, H, D):
            self._pushed = PushedOutput(B, N, H, D, dtype, device, self.group, self.timeout_ms)
        return self._pushed

    def _call_push(self, Q, K, V):
        from .ops import AnchorAttnCall
        B, h, N, D = Q.shape
        W, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        H = W * h
        pushed = self._pushed_output(B, N, H, D, Q.dtype, Q.device)
        buf, ptrs = pushed.next()
        mine = buf[:, :, rank * h:(rank + 1) * h]                       # this rank's heads inside the copy
        call = AnchorAttnCall(Q, K, V, self.sm_scale, self.block_size, self.step, self.difference,
                              out=mine.permute(0, 2, 1, 3))
        call.step1()
        call.step2()
        head_off = rank * h * D * buf.element_size()
        call.step3_push([p + head_off for p in ptrs])
        pushed.barrier()
        self.last_call = call
        return buf

    def check_status(self):
        """Synchronises; raises if a bounded device-side wait of the last call gave up (inside the
        kernels, or in the barrier because a peer never arrived)."""
        self.last_call.check_status()
        if self._pushed is not None:
            self._pushed.check_status()

    def host_call(self, Q, K, V, out):
        """The layer for tensors in pinned HOST memory: Q [B,h,N,D], K/V [B,hkv,N,D] (this rank's
        heads) in, ``out`` [B,h,N,D] (this rank's heads of the result) back in host memory; also
        returns the assembled [B,N,H,D] output on the device.  The rank's query heads are
        streamed: K/V of a KV group once, then query head by query head -- while head j computes,
        head j+1 is copied in and the result of head j-1 is copied out, each on its own CUDA
        stream.  With ``exchange="push"`` every head's rows go into all ranks' copies as they are
        computed and one barrier ends the call; with "all_gather" the heads are gathered after
        the last one.  Same bits as the device call."""
        from .ops import AnchorAttnCall
        assert not Q.is_cuda and not K.is_cuda and not V.is_cuda and not out.is_cuda, "host_call takes host tensors"
        B, h, N, D = Q.shape
        hkv = K.shape[1]
        g = h // hkv
        dev = torch.device("cuda", torch.cuda.current_device())
        multi = dist.is_initialized() and dist.get_world_size(self.group) > 1
        W, rank = (dist.get_world_size(self.group), dist.get_rank(self.group)) if multi else (1, 0)
        push = multi and self.exchange == "push"
        key = (B, h, hkv, N, D, Q.dtype)
        if self._host is None or self._host["key"] != key:
            self._host = {
                "key": key, "s_in": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev),
                "q": [torch.empty((B, 1, N, D), dtype=Q.dtype, device=dev) for _ in range(2)],
                "k": [torch.empty((B, 1, N, D), dtype=Q.dtype, device=dev) for _ in range(2)],
                "v": [torch.empty((B, 1, N, D), dtype=Q.dtype, device=dev) for _ in range(2)],
            }
        st = self._host
        s_in, s_out = st["s_in"], st["s_out"]
        main = torch.cuda.current_stream(dev)
        if push:
            pushed = self._pushed_output(B, N, W * h, D, Q.dtype, dev)
            buf, ptrs = pushed.next()
            local = buf[:, :, rank * h:(rank + 1) * h]                  # [B,N,h,D] inside the assembled copy
        else:
            if self._local is None or self._local.shape != (B, N, h, D):
                self._local = torch.empty((B, N, h, D), dtype=Q.dtype, device=dev)
                self._gathered = torch.empty((W, B, N, h, D), dtype=Q.dtype, device=dev) if W > 1 else None
            local = self._local
        q_loaded = [torch.cuda.Event() for _ in range(h)]
        kv_loaded = [torch.cuda.Event() for _ in range(hkv)]
        computed = [torch.cuda.Event() for _ in range(h)]

        def copy_in(j):
            with torch.cuda.stream(s_in):
                if j % g == 0:                                        # first head of a KV group: its K and V
                    kv = j // g
                    if kv >= 2:
                        s_in.wait_event(computed[(kv - 1) * g - 1])   # last user of this K/V buffer (group kv-2)
                    st["k"][kv & 1].copy_(K[:, kv:kv + 1], non_blocking=True)
                    st["v"][kv & 1].copy_(V[:, kv:kv + 1], non_blocking=True)
                    kv_loaded[kv].record(s_in)
                if j >= 2:
                    s_in.wait_event(computed[j - 2])                  # the query buffer's previous user
                st["q"][j & 1].copy_(Q[:, j:j + 1], non_blocking=True)
                q_loaded[j].record(s_in)

        s_in.wait_stream(main)
        s_out.wait_stream(main)
        copy_in(0)
        for j in range(h):
            if j + 1 < h:
                copy_in(j + 1)
            kv = j // g
            main.wait_event(kv_loaded[kv])
            main.wait_event(q_loaded[j])
            call = AnchorAttnCall(st["q"][j & 1], st["k"][kv & 1], st["v"][kv & 1], self.sm_scale, self.block_size,
                                  self.step, self.difference, out=local[:, :, j:j + 1].permute(0, 2, 1, 3))
            call.step1()
            call.step2()
            if push:
                head_off = (rank * h + j) * D * buf.element_size()
                call.step3_push([p + head_off for p in ptrs])
            else:
                call.step3()
            computed[j].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[j])
                out[:, j].copy_(local[:, :, j], non_blocking=True)
        self.last_call = call
        if push:
            pushed.barrier()
            full = buf
        elif W > 1:
            full = gather_heads(local, self.group, self._gathered)
        else:
            full = local
        main.wait_stream(s_out)
        main.synchronize()
        return full

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
