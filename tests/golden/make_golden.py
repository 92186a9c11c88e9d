"""Generate golden vectors by running the reference's own kernels.

    python tests/golden/make_golden.py --ref-root <checkout of the reference> [--out tests/golden]

Without a GPU the reference's Triton kernels are executed by Triton's CPU
interpreter (TRITON_INTERPRET=1), which supports fp16 but not bf16, so those
fixtures are fp16 (files ``ref_interp_fp16_*.npz``).  With a GPU the kernels are
JIT-compiled and run in bf16 (files ``ref_gpu_bf16_*.npz``).

The inputs are not stored: they are regenerated from the seed by
``oracle.anchor_oracle.make_inputs``; a checksum of the inputs is stored so a
drift in the generator is detected.  Stored per case: counts, the concatenated
id lists, M, L, a row subsample of Acc, and the operator output (fp16 values for the
interpreter fixtures, raw bf16 bit patterns as int16 for the GPU fixtures).

The reference functions called are ``anchor_attn_step_1`` / ``anchor_attn_step_2``
(anchor_attn/src/ops/anchor_step_1_2_v2.py:164-210) and ``anchor_attn``
(anchor_attn/src/ops/anchor_attn_v4.py:291-324).
"""
import argparse
import hashlib
import os
import sys
import time

import numpy as np

CASES = [
    # name, N, H, Hkv, theta, rope, q_shift, seed, block_size
    ("n4096_h2_t12", 4096, 2, 1, 12.0, False, 0.0, 0, 128),
    ("n6144_h1_t11_shift", 6144, 1, 1, 11.0, False, 0.5, 1, 128),
    ("n6144_h2_t10_shift_rope", 6144, 2, 1, 10.0, True, 0.5, 2, 128),
    ("n3072_h2_t10_shift_bs64", 3072, 2, 1, 10.0, True, 0.5, 3, 64),
    ("n8192_h1_t10_shift_bs256", 8192, 1, 1, 10.0, True, 0.5, 4, 256),
]


def checksum(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(-1).view(dtype=__import__("torch").int16).numpy().tobytes())
    return h.hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", required=True)
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--cases", default="")
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
    sys.path.insert(0, os.path.abspath(args.ref_root))
    os.makedirs(args.workdir, exist_ok=True)
    os.chdir(args.workdir)          # the reference's logger creates ./log

    from oracle.anchor_oracle import make_inputs, LOG2E
    from anchor_attn.src.ops.anchor_step_1_2_v2 import anchor_attn_step_1, anchor_attn_step_2
    from anchor_attn.src.ops.anchor_attn_v4 import anchor_attn

    dtype = torch.bfloat16 if gpu else torch.float16
    dev = "cuda" if gpu else "cpu"
    tag = "ref_gpu_bf16" if gpu else "ref_interp_fp16"
    want = set(filter(None, args.cases.split(",")))
    for name, N, H, Hkv, theta, rope, q_shift, seed, block in CASES:
        if want and name not in want:
            continue
        t0 = time.time()
        Q, K, V = make_inputs(N, H, Hkv, seed=seed, rope=rope, dtype=dtype, q_shift=q_shift)
        csum = checksum(Q, K, V)
        g = H // Hkv
        Qd = Q.to(dev)
        Kd = K.repeat_interleave(g, dim=1).to(dev).contiguous()   # what repeat_kv yields
        Vd = V.repeat_interleave(g, dim=1).to(dev).contiguous()
        B, _, _, D = Q.shape
        sm_scale = 1.0 / (D ** 0.5)
        L, M, Acc = anchor_attn_step_1(Qd, Kd, Vd, 1, 1, block, 16, B, H, N, D, sm_scale, 128, 128)
        coords, counts = anchor_attn_step_2(Qd, Kd, M, block, 16, theta * LOG2E, B, H, N, D, sm_scale)
        out, ratio = anchor_attn(Qd, Kd, Vd, None, block, 16, theta, True)
        counts = counts.cpu().numpy()[0, :, :, 0]                 # [H, NB]
        coords = coords.cpu().numpy()[0]                          # [H, NB, N]
        flat = np.concatenate([coords[h, b, :counts[h, b]] for h in range(H) for b in range(N // (block * 16))]
                              or [np.zeros(0, np.int32)]).astype(np.int32)
        np.savez_compressed(
            os.path.join(args.out, f"{tag}_{name}.npz"),
            N=N, H=H, Hkv=Hkv, theta=theta, rope=rope, q_shift=q_shift, seed=seed, block=block,
            inputs_sha256=csum, counts=counts, ids=flat,
            M=M.float().cpu().numpy()[0], L=L.float().cpu().numpy()[0],
            Acc_rows16=Acc.float().cpu().numpy()[0, :, ::16],
            out=(out.view(torch.int16).cpu().numpy()[0] if gpu else out.float().cpu().numpy()[0].astype(np.float16)),
            ratio=float(ratio),
        )
        print(f"{name}: counts sum {counts.sum()} ratio {float(ratio):.4f} in {time.time() - t0:.1f}s", flush=True)


if __name__ == "__main__":
    main()
