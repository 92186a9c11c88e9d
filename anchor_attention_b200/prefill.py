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

With N > 1 GPUs every rank holds the whole model; the attention of each layer is
computed head-parallel (each rank its KV-head groups, one all-gather of the head
outputs), the dense layers are replicated.  Prints one JSON line on rank 0.
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


def prefill_once(model, ids):
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
    if args.attn == "anchor_attn":
        patch.patch_model(model, "anchor_attn", {"theta": args.theta})
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
        logits = prefill_once(model, ids)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        logits = prefill_once(model, ids)
    e1.record()
    barrier()
    t_wall = (time.perf_counter() - t_wall) / args.steps
    ms = e0.elapsed_time(e1) / args.steps
    if W > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    if rank == 0:
        n_params = sum(p.numel() for p in model.parameters())
        print(json.dumps({
            "metric": "whole_model_prefill_latency", "value": ms, "unit": "ms", "n_gpus": W, "steps": args.steps,
            "warmup": args.warmup, "wall_ms": t_wall * 1e3, "attention": args.attn,
            "config": {"model": f"Llama-3.1-8B architecture, random init, {args.layers} layers", "seq_len": args.seq,
                       "params": n_params, "theta": args.theta, "dtype": "bf16",
                       "parallelism": "attention head-parallel, dense layers replicated" if W > 1 else "single GPU"},
            "tokens_per_s": args.seq / (ms * 1e-3), "logits_finite": bool(torch.isfinite(logits.float()).all()),
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
        }), flush=True)
    if W > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
