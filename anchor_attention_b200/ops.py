"""Host side of the operator: the reference's ``anchor_attn`` entry point backed by
the CUDA library through its C ABI.

Mirrors ``anchor_attn`` of the reference (anchor_attn/src/ops/anchor_attn_v4.py:291-324):
same name, positional/keyword signature, defaults, assertions and return
convention.  In addition K and V may carry fewer heads than Q (grouped-query
attention); query head h then reads KV head ``h // (H // Hkv)``, which is what
the reference's caller obtains by expanding K/V with ``repeat_kv`` first
(anchor_attn/src/modules/llama/anchor_attention.py:89-91).

PyTorch is used for device memory and the current stream only.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib

__all__ = ["anchor_attn", "anchor_attn_without_anchor", "anchor_attn_test_time", "anchor_attn_host",
           "AnchorAttnCall", "dense_causal_attention", "launches_per_forward"]

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_NVTX = os.environ.get("ANCHOR_ATTN_NVTX", "0") == "1"


def _workspace(device: torch.device, stream_id: int, nbytes: int) -> torch.Tensor:
    """One scratch buffer per (device, stream), grown on demand and reused."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_id)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        _workspaces.pop(key, None)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _usable(t: torch.Tensor) -> torch.Tensor:
    """The kernels take any [B,h,N,D] view whose D axis is contiguous and whose
    other strides and base address are 16-byte multiples; anything else is copied."""
    ok = t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


class AnchorAttnCall:
    """One prepared operator call: validated shapes, the parameter block and
    typed views of the workspace.  ``run()`` enqueues the whole operator;
    ``step1()``, ``step2()``, ``step3()`` enqueue one step each (used by tests to
    look at the intermediate state)."""

    def __init__(self, Q, K, V, sm_scale=None, block_size=128, step=16, difference=12.0,
                 out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                 gather_scratch_bytes: Optional[int] = None):
        """``gather_scratch_bytes``: size of the scratch step 3 copies the selected K/V rows of
        non-contiguous id tiles into (64 KB per tile).  None = the library's recommendation
        (every tile, at most 8 GiB); 0 = none, every CTA gathers its rows itself.  Ignored when
        ``workspace`` is given (its size decides)."""
        lib = _lib.load()
        assert Q.dim() == 4 and K.dim() == 4 and V.dim() == 4, "Q, K, V must be [B, H, N, D]"
        assert Q.is_cuda and K.is_cuda and V.is_cuda, "Q, K, V must be CUDA tensors (there is no CPU path)"
        assert Q.dtype == torch.bfloat16 and K.dtype == Q.dtype and V.dtype == Q.dtype, \
            "Q, K, V must be bfloat16"
        assert step in [16, 32], \
            f"Invalid step size: {step}. Only step sizes 16 or 32 are supported."
        assert block_size in (64, 128, 256), f"block_size {block_size} is not supported (64, 128 or 256)"
        assert Q.size(-2) % (block_size * step) == 0, \
            f"Sequence length {Q.size(-2)} must be divisible by (block_size * step = {block_size * step})."
        B, H, N, D = Q.shape
        Hkv = K.shape[1]
        assert D == 128, f"head dimension {D} is not supported (128 only)"
        assert K.shape == V.shape and K.shape[0] == B and K.shape[2] == N and K.shape[3] == D, \
            "K and V must be [B, Hkv, N, D] with the batch, length and head size of Q"
        assert H % Hkv == 0, f"{Hkv} KV heads do not divide {H} query heads"
        self.Q, self.K, self.V = _usable(Q), _usable(K), _usable(V)
        self.out = out if out is not None else torch.empty((B, H, N, D), dtype=Q.dtype, device=Q.device)
        self.B, self.H, self.Hkv, self.N, self.D = B, H, Hkv, N, D
        self.block_size, self.step = block_size, step
        self.NB = N // (block_size * step)
        p = _lib.AAParams()
        p.B, p.H, p.Hkv, p.N, p.D = B, H, Hkv, N, D
        p.block_size, p.step, p.dtype = block_size, step, _lib.AA_BF16
        p.theta = float(difference)
        p.sm_scale = float(sm_scale) if sm_scale else 0.0
        p.q, p.k, p.v, p.out = self.Q.data_ptr(), self.K.data_ptr(), self.V.data_ptr(), self.out.data_ptr()
        for name, t in (("q", self.Q), ("k", self.K), ("v", self.V), ("o", self.out)):
            setattr(p, f"{name}_stride_b", t.stride(0))
            setattr(p, f"{name}_stride_h", t.stride(1))
            setattr(p, f"{name}_stride_n", t.stride(2))
        lay = _lib.AALayout()
        rc = lib.aa_workspace_layout(ctypes.byref(p), ctypes.byref(lay))
        if rc != _lib.AA_OK:
            raise AssertionError(_lib.error_text(rc))
        self.layout = lay
        self.stream = torch.cuda.current_stream(Q.device)
        if workspace is None:
            nbytes = lay.total_bytes if gather_scratch_bytes is None else lay.min_bytes + int(gather_scratch_bytes)
            workspace = _workspace(Q.device, self.stream.cuda_stream, nbytes)
        self.workspace = workspace
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel()
        self.params = p
        self._lib = lib

    # ---- launches -------------------------------------------------------
    def _call(self, fn, label=None):
        """Enqueue one entry point; with ANCHOR_ATTN_NVTX=1 the launch is wrapped in an NVTX
        range named after the step, so that a timeline shows the three steps of every call."""
        nvtx = label is not None and _NVTX
        if nvtx:
            torch.cuda.nvtx.range_push(label)
        try:
            with torch.cuda.device(self.Q.device):
                rc = fn(ctypes.byref(self.params), ctypes.c_void_p(self.stream.cuda_stream))
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()
        if rc != _lib.AA_OK:
            raise RuntimeError(f"anchor_attn: {_lib.error_text(rc)}")

    def run(self):
        if _NVTX:                      # one range per step instead of one for the whole call
            self.step1()
            self.step2()
            return self.step3()
        self._call(self._lib.aa_forward)
        return self.out

    def step1(self):
        self._call(self._lib.aa_step1_anchor, "anchor_attn.step1_anchor")

    def step2(self):
        self._call(self._lib.aa_step2_stripes, "anchor_attn.step2_stripes")

    def step3(self):
        self._call(self._lib.aa_step3_sparse, "anchor_attn.step3_sparse")
        return self.out

    def step3_push(self, peer_ptrs, rows_per_peer: int = 0):
        """Step 3 that stores every output row to each address in ``peer_ptrs`` (device
        pointers with this call's output strides; may be other GPUs' memory) instead of
        ``self.out``.  With ``rows_per_peer`` > 0 row n goes only to ``peer_ptrs[n // rows_per_peer]``
        (at row ``n % rows_per_peer`` there): the token-sharded output of a sequence-parallel
        model.  Used by the head-parallel wrappers."""
        push = _lib.AAPush()
        push.n_peers = len(peer_ptrs)
        push.rows_per_peer = int(rows_per_peer)
        for i, ptr in enumerate(peer_ptrs):
            push.out[i] = ptr
        with torch.cuda.device(self.Q.device):
            rc = self._lib.aa_step3_sparse_push(ctypes.byref(self.params), ctypes.byref(push),
                                                ctypes.c_void_p(self.stream.cuda_stream))
        if rc != _lib.AA_OK:
            raise RuntimeError(f"anchor_attn: {_lib.error_text(rc)}")

    def check_status(self):
        self._call(self._lib.aa_check_status)

    def validate_lists(self):
        """Enqueue the read-only check of the id lists in the workspace (counts within capacity,
        ids ascending and inside the candidate range); ``check_status()`` then raises if a list is
        malformed.  For callers that fill or keep the lists themselves before ``step3()``."""
        self._call(self._lib.aa_validate_lists)

    @property
    def launches(self) -> int:
        """Kernels of the library one ``run()`` of this call enqueues (step 3 enqueues both of its
        sequences when the gather scratch has no slot for every possible tile)."""
        n = _lib.load().aa_forward_launches(ctypes.byref(self.params))
        if n < 0:
            raise RuntimeError(f"aa_forward_launches: {_lib.error_text(-n)}")
        return n

    @property
    def gather_slots_used(self) -> int:
        """64 KB gather slots step 3 handed out in its last run (synchronises); when that run went KV head
        by KV head (status word 4), those of its last part."""
        return int(self._view(self.layout.status_off, 4, torch.int32)[2])

    # ---- typed views of the workspace ----------------------------------
    def _view(self, off, count, dtype):
        size = torch.empty((), dtype=dtype).element_size()
        return self.workspace[off: off + count * size].view(dtype)

    @property
    def M(self):
        return self._view(self.layout.m_off, self.B * self.H * self.N, torch.float32).view(self.B, self.H, self.N)

    @property
    def L(self):
        return self._view(self.layout.l_off, self.B * self.H * self.N, torch.float32).view(self.B, self.H, self.N)

    @property
    def Acc(self):
        """Step 1's un-normalised output as a [B,H,N,D] tensor (a copy).  In the workspace it is kept
        in tiles of 128 rows, each tile chunk-major: [B, H, N/128, D/4 chunks, 128 rows, 4]."""
        raw = self._view(self.layout.acc_off, self.B * self.H * self.N * self.D, torch.float32).view(
            self.B, self.H, self.N // 128, self.D // 4, 128, 4)
        return raw.permute(0, 1, 2, 4, 3, 5).reshape(self.B, self.H, self.N, self.D)

    @property
    def qpool(self):
        n = self.N // self.block_size
        return self._view(self.layout.qpool_off, self.B * self.H * n * self.D, torch.bfloat16).view(
            self.B, self.H, n, self.D)

    @property
    def apool(self):
        n = self.N // self.block_size
        return self._view(self.layout.apool_off, self.B * self.H * n, torch.float32).view(self.B, self.H, n)

    @property
    def counts(self):
        return self._view(self.layout.counts_off, self.B * self.H * self.NB, torch.int32).view(
            self.B, self.H, self.NB)

    @property
    def ids(self):
        return self._view(self.layout.ids_off, self.B * self.H * self.layout.ids_per_head, torch.int32).view(
            self.B, self.H, self.layout.ids_per_head)

    def id_row_offset(self, b: int) -> int:
        return self._lib.aa_id_row_offset(self.block_size, self.step, b)

    def id_lists(self) -> List[List[List[torch.Tensor]]]:
        """[B][H][NB] ascending int32 id tensors on the CPU (synchronises)."""
        counts = self.counts.cpu()
        ids = self.ids.cpu()
        return [[[ids[z, h, self.id_row_offset(b): self.id_row_offset(b) + int(counts[z, h, b])].clone()
                  for b in range(self.NB)] for h in range(self.H)] for z in range(self.B)]

    def coords_reference_layout(self):
        """(true_coords [B,H,NB,N], true_counts [B,H,NB,1]) as the reference's
        step 2 returns them (get_mask_test.py:138-145); slots past the count are 0."""
        coords = torch.zeros((self.B, self.H, self.NB, self.N), dtype=torch.int32, device=self.Q.device)
        counts = self.counts
        for b in range(1, self.NB):
            cap = b * self.block_size * self.step - 2 * self.block_size
            off = self.id_row_offset(b)
            seg = self.ids[:, :, off: off + cap]
            keep = torch.arange(cap, device=seg.device)[None, None, :] < counts[:, :, b: b + 1]
            coords[:, :, b, :cap] = torch.where(keep, seg, torch.zeros_like(seg))
        return coords, counts.unsqueeze(-1).clone()

    def ratio(self) -> torch.Tensor:
        """anchor_attn_v4.py:271."""
        denom = (self.B * self.H * self.N * self.N / (self.block_size * self.step)) // 2
        return self.counts.sum() / denom


def anchor_attn(Q, K, V,
                sm_scale: float = None,
                block_size: int = 128,
                step: int = 16,
                difference: float = 12,
                return_computational_ratio: bool = True):
    """Anchor attention prefill.  Q [B,H,N,D]; K, V [B,H,N,D] or [B,Hkv,N,D]; bf16.
    Returns ``(out, ratio)`` or ``out`` exactly like the reference operator
    (anchor_attn/src/ops/anchor_attn_v4.py:291-324); ``out`` is a new [B,H,N,D]
    tensor.  The launches are asynchronous on the current CUDA stream."""
    call = AnchorAttnCall(Q, K, V, sm_scale, block_size, step, difference)
    out = call.run()
    if return_computational_ratio:
        return out, call.ratio()
    return out


def anchor_attn_without_anchor(Q, K, V,
                               sm_scale: float = None,
                               block_size: int = 128,
                               step: int = 16,
                               difference: float = 12):
    """The reference's second entry point (anchor_attn/src/ops/anchor_attn_v4.py:275-289,
    171-224): the same three steps with the same arithmetic as ``anchor_attn``; it always
    returns ``(out, sparsity_ratio)``."""
    return anchor_attn(Q, K, V, sm_scale, block_size, step, difference, return_computational_ratio=True)


def anchor_attn_test_time(Q, K, V,
                          sm_scale: float = None,
                          block_size: int = 128,
                          step: int = 16,
                          difference: float = 12,
                          return_computational_ratio: bool = True):
    """The reference's timing entry point (anchor_attn/src/ops/anchor_attn_v4.py:328-354, 107-169):
    the same operator with the host synchronised around the search phase (steps 1 and 2) and the
    compute phase (step 3), wall-clock milliseconds of each returned after the output.  Returns
    ``(out, ratio, search_ms, compute_ms)`` or ``(out, search_ms, compute_ms)``."""
    import time
    call = AnchorAttnCall(Q, K, V, sm_scale, block_size, step, difference)
    torch.cuda.synchronize(Q.device)
    t0 = time.time()
    call.step1()
    call.step2()
    torch.cuda.synchronize(Q.device)
    search_ms = (time.time() - t0) * 1000
    t0 = time.time()
    out = call.step3()
    torch.cuda.synchronize(Q.device)
    compute_ms = (time.time() - t0) * 1000
    if return_computational_ratio:
        return out, call.ratio(), search_ms, compute_ms
    return out, search_ms, compute_ms


def anchor_attn_host(Q, K, V, out=None,
                     sm_scale: float = None,
                     block_size: int = 128,
                     step: int = 16,
                     difference: float = 12,
                     device=None):
    """``anchor_attn`` for tensors that live in (pinned) host memory: Q [B,H,N,D], K/V
    [B,Hkv,N,D] bf16 on the CPU in, ``out`` [B,H,N,D] on the CPU out (allocated pinned if
    not given).  The KV-head groups are independent, so they are streamed: while one chunk
    of query heads computes on the device, the next chunk is copied in and the result of
    the previous one is copied out, each on its own CUDA stream.  A chunk is a whole KV
    group, except that the first and the last group go head by head, so that the first
    computation starts after one head's worth of queries (plus its K/V) has arrived and only
    one head's output is left to copy when the last computation ends.  The call returns once
    ``out`` is complete.  Same arithmetic, head by head, as ``anchor_attn`` on device tensors."""
    assert not Q.is_cuda and not K.is_cuda and not V.is_cuda, "anchor_attn_host takes host tensors"
    B, H, N, D = Q.shape
    Hkv = K.shape[1]
    assert H % Hkv == 0, f"{Hkv} KV heads do not divide {H} query heads"
    Hg = H // Hkv
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    if out is None:
        out = torch.empty((B, H, N, D), dtype=Q.dtype).pin_memory()
    # chunks: (KV group, first query head, number of heads)
    chunks = []
    for g in range(Hkv):
        if g in (0, Hkv - 1) and Hg > 1:
            chunks += [(g, g * Hg + i, 1) for i in range(Hg)]
        else:
            chunks.append((g, g * Hg, Hg))
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dq = [torch.empty((B, Hg, N, D), dtype=Q.dtype, device=dev) for _ in range(2)]
    do = [torch.empty((B, Hg, N, D), dtype=Q.dtype, device=dev) for _ in range(2)]
    dk = [torch.empty((B, 1, N, D), dtype=Q.dtype, device=dev) for _ in range(2)]
    dv = [torch.empty((B, 1, N, D), dtype=Q.dtype, device=dev) for _ in range(2)]
    n = len(chunks)
    loaded = [torch.cuda.Event() for _ in range(n)]
    computed = [torch.cuda.Event() for _ in range(n)]
    drained = [torch.cuda.Event() for _ in range(n)]
    last_chunk_of_group = {g: max(c for c, ch in enumerate(chunks) if ch[0] == g) for g in range(Hkv)}

    def copy_in(c):
        g, h0, nh = chunks[c]
        with torch.cuda.stream(s_in):
            if c == 0 or chunks[c - 1][0] != g:                  # first chunk of its group: the group's K and V
                if g >= 2:
                    s_in.wait_event(computed[last_chunk_of_group[g - 2]])   # the K/V buffer's previous user
                dk[g & 1].copy_(K[:, g:g + 1], non_blocking=True)
                dv[g & 1].copy_(V[:, g:g + 1], non_blocking=True)
            if c >= 2:
                s_in.wait_event(computed[c - 2])                 # the query buffer's previous user
            dq[c & 1][:, :nh].copy_(Q[:, h0:h0 + nh], non_blocking=True)
            loaded[c].record(s_in)

    s_in.wait_stream(main)
    copy_in(0)
    for c, (g, h0, nh) in enumerate(chunks):
        if c + 1 < n:
            copy_in(c + 1)
        main.wait_event(loaded[c])
        if c >= 2:
            main.wait_event(drained[c - 2])                      # the output buffer has been copied out
        AnchorAttnCall(dq[c & 1][:, :nh], dk[g & 1], dv[g & 1], sm_scale, block_size, step, difference,
                       out=do[c & 1][:, :nh]).run()
        computed[c].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(computed[c])
            out[:, h0:h0 + nh].copy_(do[c & 1][:, :nh], non_blocking=True)
            drained[c].record(s_out)
    main.wait_stream(s_out)
    main.synchronize()
    return out


_dense_status: Dict[int, torch.Tensor] = {}


def dense_causal_attention(query, key, value, scaling: float = None, out: Optional[torch.Tensor] = None):
    """Dense causal attention of the LAST ``q`` positions of a ``kv``-long sequence on the library's
    own attention kernel: query [B,H,q,D], key/value [B,Hkv,kv,D] (kv >= q), bf16 CUDA tensors,
    D = 128; row i attends keys 0 .. kv - q + i.  Returns [B,H,q,D] (``out`` may be a strided view,
    e.g. of token-major memory).  The path the reference sends to flash-attn for the tail of a
    prefill and for later chunks (anchor_attn/src/modules/llama/anchor_attention.py:76-88, 101-113).
    A prefill kernel (128-row tiles): single-token decode should keep using a split-KV library kernel."""
    lib = _lib.load()
    assert query.is_cuda and key.is_cuda and value.is_cuda, "dense_causal_attention takes CUDA tensors (no CPU path)"
    assert query.dtype == torch.bfloat16 and key.dtype == query.dtype and value.dtype == query.dtype
    B, H, nq, D = query.shape
    Hkv, nkv = key.shape[1], key.shape[2]
    assert D == 128 and key.shape == value.shape and key.shape[0] == B and key.shape[3] == D
    assert H % Hkv == 0 and nkv >= nq >= 1
    q, k, v = _usable(query), _usable(key), _usable(value)
    if out is None:
        out = torch.empty((B, H, nq, D), dtype=query.dtype, device=query.device)
    dev = query.device.index if query.device.index is not None else torch.cuda.current_device()
    status = _dense_status.get(dev)
    if status is None:
        status = _dense_status[dev] = torch.zeros(4, dtype=torch.int32, device=query.device)
    a = _lib.AADenseCausal()
    a.B, a.H, a.Hkv, a.Nq, a.Nkv, a.D = B, H, Hkv, nq, nkv, D
    a.dtype = _lib.AA_BF16
    a.sm_scale = float(scaling) if scaling else 0.0
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    for name, t in (("q", q), ("k", k), ("v", v), ("o", out)):
        setattr(a, f"{name}_stride_b", t.stride(0))
        setattr(a, f"{name}_stride_h", t.stride(1))
        setattr(a, f"{name}_stride_n", t.stride(2))
    a.status = status.data_ptr()
    with torch.cuda.device(query.device):
        rc = lib.aa_dense_causal_attend(ctypes.byref(a), ctypes.c_void_p(torch.cuda.current_stream(query.device).cuda_stream))
    if rc != _lib.AA_OK:
        raise RuntimeError(f"dense_causal_attention: {_lib.error_text(rc)}")
    return out


def launches_per_forward() -> int:
    """Kernels of the library one operator call enqueues, at least (see ``AnchorAttnCall.launches``)."""
    return _lib.load().aa_launches_per_forward()
