"""Whole-model prefill over several GPUs: token-parallel dense layers, head-parallel attention.

The reference runs its prefill on one GPU (test_hf.py:119-131).  Every layer of a
Llama-style decoder except attention is token-local -- embedding, RMSNorm, the q/k/v
projections with RoPE (anchor_attn/src/modules/llama/anchor_attention.py:30-48), the
output projection and the MLP (llama_mlp_forward.py:49-56) -- and anchor attention is
independent per query head.  So rank r of W

  * owns the tokens [r*N/W, (r+1)*N/W) for all token-local work (1/W of every GEMM), and
  * owns the query heads of its KV groups (``parallel.head_partition``) for attention.

Two exchanges per layer turn one partition into the other:

  tokens -> heads   the rotated q/k/v of a rank's tokens go to the ranks that own the heads
                    (each rank receives N x (h + 2 hkv) x D elements, token-major, which the
                    attention kernels read in place through their strides): one kernel
                    (``aa_rope_dispatch``) applies the rotary embedding and stores every head row
                    straight into its owner's buffer over NVLink, then the flag barrier; or, with
                    ``exchange="all_to_all"``, the library rotary function, a packing copy and one
                    all-to-all collective;
  heads -> tokens   step 3 stores every finished output row straight into the [n_loc, H, D]
                    buffer of the rank that owns the row's token (``aa_step3_sparse_push`` with
                    ``rows_per_peer``: plain stores over NVLink while the other CTAs compute),
                    followed by the bounded flag barrier; or, with ``exchange="all_to_all"``,
                    a second collective (works on any backend, used by the CPU tests).

The weights are replicated; activations and all dense FLOPs are divided by W.  Results equal
the single-GPU model's up to the rounding of GEMMs on different row counts.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from .parallel import PushedOutput, head_partition


class SequenceParallelPrefill:
    """Prefill of a Hugging Face Llama-style causal LM (``model.model.layers[i]`` with
    ``input_layernorm, self_attn.{q,k,v,o}_proj, post_attention_layernorm, mlp``) patched for
    anchor attention, over the ranks of ``group``.  Every rank passes the same ``input_ids``
    [1, N]; N must be a multiple of ``W * 256`` and of ``block_size * step``.  Returns the
    last token's logits [1, 1, vocab] on every rank.

    ``attn_fn(Q [1,h,N,D], K [1,hkv,N,D], V) -> [1,N,h,D]`` replaces the CUDA operator (the CPU
    tests pass the oracle; the exchange is then the all-to-all)."""

    def __init__(self, model, group=None, exchange: str = "push", attn_fn: Optional[Callable] = None,
                 timeout_ms: int = 10000):
        if exchange not in ("push", "all_to_all"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.model = model
        self.group = group if group is not None else dist.group.WORLD
        self.W, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.exchange = "all_to_all" if attn_fn is not None else exchange
        self.attn_fn = attn_fn
        self.timeout_ms = timeout_ms
        cfg = model.config
        self.H, self.Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.D = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.block, self.step, self.theta = int(cfg.block_size_M), int(cfg.step), float(cfg.theta)
        self.q_lo, self.q_hi, self.kv_lo, self.kv_hi = head_partition(self.H, self.Hkv, self.W, self.rank)
        self._pushed = None
        self._qkv = None
        self.last_call = None
        self.profile = False          # True: the next call records CUDA events between the stages of every layer
        self.stage_ms = {}            # stage -> milliseconds summed over the layers of the last profiled call

    def _mark(self, marks, name):
        if marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    # ---- exchanges --------------------------------------------------------------------
    def _tokens_to_heads(self, q, k, v):
        """q [1,n,H,D], k/v [1,n,Hkv,D] of this rank's tokens -> (Q [1,h,N,D], K [1,hkv,N,D], V)
        of this rank's heads over all tokens, as strided views of the received buffer."""
        W, n = self.W, q.shape[1]
        h, hkv, D = self.H // W, self.Hkv // W, self.D
        send = torch.cat([q.view(1, n, W, h, D), k.view(1, n, W, hkv, D), v.view(1, n, W, hkv, D)], dim=3)
        send = send[0].permute(1, 0, 2, 3).contiguous()                    # [W, n, h+2hkv, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        recv = recv.view(1, W * n, h + 2 * hkv, D)                         # tokens in order, token-major
        Q = recv[:, :, :h].permute(0, 2, 1, 3)
        K = recv[:, :, h:h + hkv].permute(0, 2, 1, 3)
        V = recv[:, :, h + hkv:].permute(0, 2, 1, 3)
        return Q, K, V

    def _rope_dispatch(self, qp, kp, vp, cos, sin, lo):
        """The fused path of the tokens -> heads exchange: qp [1,n,H*D], kp/vp [1,n,Hkv*D] are the
        projections of this rank's tokens, cos/sin [1,n,D] their rotary tables; returns (Q, K, V) of
        this rank's heads over all tokens as strided views of its symmetric buffer."""
        import ctypes
        from . import _lib
        W, n = self.W, qp.shape[1]
        h, hkv, D = self.H // W, self.Hkv // W, self.D
        N = W * n
        if self._qkv is None or self._qkv.shape != (1, N, h + 2 * hkv, D):
            self._qkv = PushedOutput(1, N, h + 2 * hkv, D, qp.dtype, qp.device, self.group, self.timeout_ms)
        buf, ptrs = self._qkv.next()
        r = _lib.AARopeDispatch()
        r.n, r.H, r.Hkv, r.D, r.dtype = n, self.H, self.Hkv, D, _lib.AA_BF16
        r.n_peers, r.token0 = W, lo
        r.q, r.k, r.v = qp.data_ptr(), kp.data_ptr(), vp.data_ptr()
        r.q_stride_n, r.k_stride_n, r.v_stride_n = qp.stride(1), kp.stride(1), vp.stride(1)
        cos, sin = cos.contiguous(), sin.contiguous()
        r.cos, r.sin = cos.data_ptr(), sin.data_ptr()
        for i, p in enumerate(ptrs):
            r.dst[i] = p
        with torch.cuda.device(qp.device):
            rc = _lib.load().aa_rope_dispatch(ctypes.byref(r),
                                              ctypes.c_void_p(torch.cuda.current_stream(qp.device).cuda_stream))
        if rc != _lib.AA_OK:
            raise RuntimeError(f"aa_rope_dispatch: {_lib.error_text(rc)}")
        self._qkv.barrier()
        Q = buf[:, :, :h].permute(0, 2, 1, 3)
        K = buf[:, :, h:h + hkv].permute(0, 2, 1, 3)
        V = buf[:, :, h + hkv:].permute(0, 2, 1, 3)
        return Q, K, V

    def _heads_to_tokens(self, out_heads):
        """out_heads [1,N,h,D] (this rank's heads, all tokens) -> [1,n,H,D] (all heads, own tokens)."""
        W = self.W
        _, N, h, D = out_heads.shape
        n = N // W
        send = out_heads.reshape(W, n, h, D).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv.permute(1, 0, 2, 3).reshape(1, n, W * h, D)

    def _attention(self, Q, K, V, scaling, n_loc):
        """Anchor attention on this rank's heads; returns [1, n_loc, H, D] for this rank's tokens."""
        W, rank = self.W, self.rank
        _, h, N, D = Q.shape
        if self.attn_fn is not None:
            return self._heads_to_tokens(self.attn_fn(Q, K, V))
        from .ops import AnchorAttnCall
        if self.exchange == "all_to_all":
            local = torch.empty((1, N, h, D), dtype=Q.dtype, device=Q.device)
            call = AnchorAttnCall(Q, K, V, scaling, self.block, self.step, self.theta, out=local.permute(0, 2, 1, 3))
            call.run()
            self.last_call = call
            return self._heads_to_tokens(local)
        if self._pushed is None or self._pushed.shape != (1, n_loc, self.H, D):
            self._pushed = PushedOutput(1, n_loc, self.H, D, Q.dtype, Q.device, self.group, self.timeout_ms)
        buf, ptrs = self._pushed.next()
        # the call's output strides describe a [1, N, H, D] tensor; row n lands in the copy of
        # rank n // n_loc at local row n % n_loc
        dummy = buf[:, :, rank * h:(rank + 1) * h].permute(0, 2, 1, 3)      # strides only (osn = H*D, osh = D)
        call = AnchorAttnCall(Q, K, V, scaling, self.block, self.step, self.theta, out=dummy)
        call.step1()
        call.step2()
        head_off = rank * h * D * buf.element_size()
        call.step3_push([p + head_off for p in ptrs], rows_per_peer=n_loc)
        self._pushed.barrier()
        self.last_call = call
        return buf

    # ---- the model ----------------------------------------------------------------------
    @torch.no_grad()
    def __call__(self, input_ids: torch.Tensor) -> torch.Tensor:
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
        model, W, rank = self.model, self.W, self.rank
        N = input_ids.shape[1]
        G = self.block * self.step
        if input_ids.shape[0] != 1 or N % (W * 256) != 0 or N % G != 0:
            raise ValueError(f"sequence-parallel prefill needs batch 1 and a length that is a multiple of "
                             f"{W * 256} and of block_size*step = {G}; got {tuple(input_ids.shape)}")
        n = N // W
        lo = rank * n
        base = model.model
        x = base.embed_tokens(input_ids[:, lo:lo + n])
        pos = torch.arange(lo, lo + n, device=x.device)[None]
        cos, sin = base.rotary_emb(x, position_ids=pos)
        H, Hkv, D = self.H, self.Hkv, self.D
        fused = (self.attn_fn is None and self.exchange == "push" and x.is_cuda and x.dtype == torch.bfloat16
                 and D == 128)
        marks = [] if (self.profile and x.is_cuda) else None
        self._mark(marks, "start")
        for layer in base.layers[: model.config.num_hidden_layers]:
            attn = layer.self_attn
            hn = layer.input_layernorm(x)
            qp, kp, vp = attn.q_proj(hn), attn.k_proj(hn), attn.v_proj(hn)
            if fused:
                self._mark(marks, "norm_qkv")
                Q, K, V = self._rope_dispatch(qp, kp, vp, cos, sin, lo)
                self._mark(marks, "rope_and_tokens_to_heads")
            else:
                q = qp.view(1, n, H, D).transpose(1, 2)
                k = kp.view(1, n, Hkv, D).transpose(1, 2)
                q, k = apply_rotary_pos_emb(q, k, cos, sin)
                self._mark(marks, "norm_qkv_rope")
                Q, K, V = self._tokens_to_heads(q.transpose(1, 2), k.transpose(1, 2), vp.view(1, n, Hkv, D))
                self._mark(marks, "tokens_to_heads")
            out = self._attention(Q, K, V, attn.scaling, n)                 # [1, n, H, D]
            self._mark(marks, "attention_and_heads_to_tokens")
            x = x + attn.o_proj(out.reshape(1, n, H * D))
            x = x + layer.mlp(layer.post_attention_layernorm(x))
            self._mark(marks, "o_proj_mlp")
        if marks is not None:
            torch.cuda.synchronize()
            self.stage_ms = {}
            for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                self.stage_ms[name] = self.stage_ms.get(name, 0.0) + a.elapsed_time(b)
        logits = None
        vocab = model.config.vocab_size
        if rank == W - 1:
            logits = model.lm_head(base.norm(x[:, -1:])).float().contiguous()
        else:
            logits = torch.empty((1, 1, vocab), dtype=torch.float32, device=x.device)
        dist.broadcast(logits, src=dist.get_global_rank(self.group, W - 1), group=self.group)
        return logits

    def check_status(self):
        """Synchronises; raises if a bounded device-side wait gave up (kernels or barrier)."""
        if self.last_call is not None:
            self.last_call.check_status()
        if self._pushed is not None:
            self._pushed.check_status()
        if self._qkv is not None:
            self._qkv.check_status()
