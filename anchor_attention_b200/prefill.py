"""Whole-model prefill with anchor attention in every layer.

Counterpart of the reference's quick-start harness (test_hf.py:24-36,119-131:
load a Hugging Face causal LM, ``patch_model(model, "anchor_attn", config)``,
time the prefill), for a random-init model of a given architecture -- there
are no checkpoints on the benchmark machine -- on uniform-random token ids.

    python -m anchor_attention_b200.prefill [--seq 131072] [--layers 32] [--attn anchor_attn|sdpa]
    python -m torch.distributed.run --nproc-per-node 8 -m anchor_attention_b200.prefill --gpus 8

The two memory measures the reference applies with every pattern are kept: the
language-model head runs on the last token only
(anchor_attn/src/modules/llama/causal_model_forward.py:124; here the model's own
``logits_to_keep=1``) and the MLP runs in 32768-token chunks
(llama_mlp_forward.py:49-56; ``patch_model`` installs it).

With N > 1 GPUs every rank holds the whole model.  ``--parallel seq`` (default): the dense
layers run on each rank's share of the tokens and attention on its share of the heads
(``seq_parallel.SequenceParallelPrefill``: one all-to-all in, output rows pushed to the token
owners by step 3).  ``--parallel replicated``: every rank runs all dense layers on all tokens
and only attention is head-parallel.  ``--check-logits`` also runs the single-GPU model on
rank 0 and reports the largest difference of the last-token logits.  ``--profile`` adds the
per-stage split of one prefill (CUDA events, summed over the layers).  Prints one JSON line
on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def llama31_8b_config(layers: int = 32, max_pos: int = 131072):
    from transformers import LlamaConfig
    return LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       max_position_embeddings=max_pos, rope_theta=500000.0, rms_norm_eps=1e-5,
                       tie_word_embeddings=False)


def build_model(cfg, device, seed: int = 0):
    """Random-init weights created directly on the device in bf16."""
    from transformers import LlamaForCausalLM
    torch.manual_seed(seed)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    return model.eval()


def prefill_once(model, ids, seq_par=None):
    if seq_par is not None:
        return seq_par(ids)
    with torch.no_grad():
        out = model(input_ids=ids, use_cache=False, logits_to_keep=1)
    return out.logits


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--seq", type=int, default=131072)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--attn", default="anchor_attn", choices=["anchor_attn", "sdpa"])
    ap.add_argument("--theta", type=float, default=12.0)
    ap.add_argument("--parallel", default="seq", choices=["seq", "replicated"],
                    help="N > 1: token-parallel dense layers + head-parallel attention, or replicated dense layers")
    ap.add_argument("--exchange", default="push", choices=["push", "all_to_all"],
                    help="--parallel seq: how the head outputs get back to the token owners")
    ap.add_argument("--check-logits", action="store_true",
                    help="N > 1: rank 0 also runs the single-GPU model and reports the logits' difference")
    ap.add_argument("--profile", action="store_true", help="per-stage split of one prefill (CUDA events)")
    args = ap.parse_args()

    import torch.distributed as dist
    from . import patch
    W = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if W != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={W}: launch with torch.distributed.run for N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("the prefill harness needs a CUDA device: the operator has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if W > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = llama31_8b_config(args.layers, max(args.seq, 8192))
    model = build_model(cfg, dev)
    seq_par = None
    if args.attn == "anchor_attn":
        patch.patch_model(model, "anchor_attn", {"theta": args.theta})
        if W > 1 and args.parallel == "seq":
            from .seq_parallel import SequenceParallelPrefill
            seq_par = SequenceParallelPrefill(model, dist.group.WORLD, exchange=args.exchange)
        else:
            patch.set_head_parallel_group(dist.group.WORLD if W > 1 else None)
    else:
        model.config._attn_implementation = "sdpa"
        patch.install_chunked_mlp(model)
    g = torch.Generator(device="cpu").manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (1, args.seq), generator=g).to(dev)

    def barrier():
        if W > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        logits = prefill_once(model, ids, seq_par)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        logits = prefill_once(model, ids, seq_par)
    e1.record()
    barrier()
    t_wall = (time.perf_counter() - t_wall) / args.steps
    ms = e0.elapsed_time(e1) / args.steps
    if W > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    stage_ms = None
    if args.profile and seq_par is not None:
        seq_par.profile = True
        prefill_once(model, ids, seq_par)
        seq_par.profile = False
        stage_ms = seq_par.stage_ms
        barrier()
    if seq_par is not None:
        seq_par.check_status()
    logits_diff = None
    if args.check_logits and W > 1:
        # the single-GPU model on rank 0 (attention through the hook, nothing parallel)
        if rank == 0:
            patch.set_head_parallel_group(None)
            single = prefill_once(model, ids).float()
            logits_diff = {"max_abs": float((single - logits.float()).abs().max()),
                           "mean_abs": float((single - logits.float()).abs().mean()),
                           "logit_scale": float(single.abs().max())}
        barrier()
    if rank == 0:
        n_params = sum(p.numel() for p in model.parameters())
        print(json.dumps({
            "metric": "whole_model_prefill_latency", "value": ms, "unit": "ms", "n_gpus": W, "steps": args.steps,
            "warmup": args.warmup, "wall_ms": t_wall * 1e3, "attention": args.attn,
            "config": {"model": f"Llama-3.1-8B architecture, random init, {args.layers} layers", "seq_len": args.seq,
                       "params": n_params, "theta": args.theta, "dtype": "bf16",
                       "parallelism": ("single GPU" if W == 1 else
                                       f"dense layers token-parallel, attention head-parallel, output rows {args.exchange}"
                                       if seq_par is not None else "attention head-parallel, dense layers replicated")},
            "stage_ms": stage_ms, "logits_vs_single_gpu": logits_diff,
            "tokens_per_s": args.seq / (ms * 1e-3), "logits_finite": bool(torch.isfinite(logits.float()).all()),
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
        }), flush=True)
    if W > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
