"""Generate golden vectors of the block-granular comparator by running the reference's own code.

    python tests/golden/make_golden_block_sparse.py --ref-root <checkout of the reference> [--out tests/golden]

Per case the reference's index builders (plain torch; run on fp32 copies of the inputs on the
CPU so that no score ties blur the selection) give ``block_index`` and the sparsity ratio, and
the reference's Triton kernel attends on that index: without a GPU in Triton's CPU interpreter
(TRITON_INTERPRET=1; fp16, the interpreter has no bf16; file ``block_sparse_ref_interp_fp16.npz``),
with a GPU JIT-compiled in bf16 (file ``block_sparse_ref_gpu_bf16.npz``, raw bf16 bits as int16).

The inputs are regenerated from the seed by ``oracle.anchor_oracle.make_inputs`` (a checksum is
stored); of each output every fourth row is kept.  The reference functions called are ``_build_block_index``,
``_build_block_index_top_cdf``, ``_build_block_index_difference_aware`` and
``_triton_block_sparse_attention`` (anchor_attn/src/ops/block_sparse_flash_attention_v2.py:150-309,
113-144).
"""
import argparse
import hashlib
import os
import sys
import time

import numpy as np

N, H, SEED = 1024, 2, 7
# name, builder, arguments
VARIANTS = [
    ("top_k3", "top_k", dict(top_k=3)),
    ("diff_t005", "diff", dict(theta=0.0625, top_k=1000)),    # unclipped: short rows are left-padded with zeros
    ("diff_t0125_k4", "diff", dict(theta=0.125, top_k=4)),    # clipped to four blocks
    ("cdf_05", "cdf", dict(cdf_threshold=0.5)),
]


def checksum(*tensors):
    import torch
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(-1).view(dtype=torch.int16).numpy().tobytes())
    return h.hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", required=True)
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--workdir", default="/tmp/anchor_golden_work")
    args = ap.parse_args()
    args.out = os.path.abspath(args.out)
    args.ref_root = os.path.abspath(args.ref_root)

    import torch
    gpu = torch.cuda.is_available()
    if not gpu:
        os.environ["TRITON_INTERPRET"] = "1"
    repo = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
    sys.path.insert(0, repo)
    sys.path.insert(0, args.ref_root)
    os.makedirs(args.workdir, exist_ok=True)
    os.chdir(args.workdir)          # the reference's logger creates ./log

    from oracle.anchor_oracle import make_inputs
    from anchor_attn.src.ops import block_sparse_flash_attention_v2 as ref

    dtype = torch.bfloat16 if gpu else torch.float16
    dev = "cuda" if gpu else "cpu"
    Q, K, V = make_inputs(N, H, H, seed=SEED, rope=False, dtype=dtype, q_shift=0.5)
    D = Q.shape[-1]
    sm_scale = D ** -0.5
    store = dict(N=N, H=H, seed=SEED, inputs_sha256=checksum(Q, K, V), names=np.array([v[0] for v in VARIANTS]))
    Qf, Kf = Q.float(), K.float()
    seqlens = torch.full((1,), N, dtype=torch.int32, device=dev)
    for name, kind, kw in VARIANTS:
        t0 = time.time()
        if kind == "top_k":
            idx, ratio = ref._build_block_index(Qf, Kf, kw["top_k"])
        elif kind == "cdf":
            idx, ratio = ref._build_block_index_top_cdf(Qf, Kf, kw["cdf_threshold"], 128, 128, sm_scale)
        else:
            idx, ratio = ref._build_block_index_difference_aware(Qf, Kf, 128, 128, kw["theta"], sm_scale, kw["top_k"])
        out = ref._triton_block_sparse_attention(Q.to(dev), K.to(dev), V.to(dev), seqlens, idx.to(dev), sm_scale)
        store[f"{name}_index"] = idx.cpu().numpy().astype(np.int32)
        store[f"{name}_ratio"] = float(ratio)
        # every fourth row of the output
        store[f"{name}_out"] = (out.view(torch.int16).cpu().numpy()[0, :, ::4] if gpu
                                else out.float().cpu().numpy()[0, :, ::4].astype(np.float16))
        print(f"{name}: index {tuple(idx.shape)} ratio {float(ratio):.4f} in {time.time() - t0:.1f}s", flush=True)
        print(idx[0, 0].tolist(), flush=True)
    tag = "ref_gpu_bf16" if gpu else "ref_interp_fp16"
    np.savez_compressed(os.path.join(args.out, f"block_sparse_{tag}.npz"), **store)


if __name__ == "__main__":
    main()
