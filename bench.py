#!/usr/bin/env python
"""Benchmark of the anchor-attention prefill operator (one attention layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--seq S]

Workload: one Llama-3.1-8B-shape attention layer (32 query / 8 KV heads, head
size 128, bf16, causal, batch 1) at 131072 tokens on seeded synthetic tensors
(N(0,1) entries, sink rows, 1 % stripe columns, RoPE at base 500000), block 128,
step 16, theta 12.  With N > 1 GPUs the heads are partitioned by KV group across
the ranks (strong scaling of the fixed layer); every rank ends with all head
outputs, either because step 3 stores its rows into every rank's output copy over
NVLink while it computes (default) or through one NCCL all-gather
(``--exchange all_gather``).  Prints ONE JSON line on rank 0.

``--impl reference`` times the CPU restatement of the reference operator on the
host cores on a bounded sample of the same workload and extrapolates to the
layer (the reference's own kernels are Triton GPU kernels; its "PyTorch path"
is not runnable).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, HKV, D, BLOCK, STEP, THETA = 32, 8, 128, 128, 16, 12.0
METRIC = "ms_per_layer_anchor_attn_prefill_128k_llama31_8b_heads"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one step-3 launch at density 1 on one
# GPU, from single-pass ncu captures of this benchmark (profiles/attend_tc_seq32768.md): sequence
# length -> (bytes, K/V tile-pair loads of 64 KB by all CTAs).  Other sizes, densities and per-rank
# shares are scaled from the nearest entry by their tile-pair loads.
STEP3_DRAM_CAPTURES = {32768: (1.245e9, 483840), 131072: (7.97e9, 8225280)}


def algorithmic_flops(N, H, counts_total, step=STEP):
    """FLOPs the operator must do: step 1 on causally useful pairs, step 2's pooled
    scores, step 3 on the selected columns (from the emitted counts)."""
    G = BLOCK * step
    NB = N // G
    p1 = G * (G + 1) // 2 + (NB - 1) * (G * G + G * (G + 1) // 2)
    p2 = step * sum(b * G - 2 * BLOCK for b in range(1, NB))
    f1 = 4 * D * p1 * H
    f2 = 2 * D * p2 * H
    f3 = 4 * D * G * counts_total
    return f1, f2, f3


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops_sustained"]), float(p["hbm_gbs"]), "measured"
    return 1400.0, 6650.0, "fallback"


# --------------------------------------------------------------------------
# CPU legs (the only places the oracle is executed by the benchmark)
# --------------------------------------------------------------------------
def cpu_sample(N, threads=None, limit_s=12.0):
    """Time the CPU restatement on a bounded sample of the workload: one query head
    of the N-token layer, whole big blocks (2048 query rows each, all three steps)
    taken from the last one downwards until ``limit_s`` seconds are spent, then
    scaled by the layer's query-key pair count.  Returns (extrapolated ms per
    layer, description, cores)."""
    import torch
    from oracle.anchor_oracle import oracle_big_blocks, make_inputs
    cores = threads or os.cpu_count()
    torch.set_num_threads(cores)
    Q, K, V = make_inputs(N, 1, 1, seed=0, rope=True)
    G = BLOCK * STEP
    NB = N // G
    oracle_big_blocks(Q[0, 0, :2 * G], K[0, 0, :2 * G], V[0, 0, :2 * G], [1], difference=THETA)   # warm-up
    sample_pairs, blocks, dt = 0, [], 0.0
    for b in range(NB - 1, -1, -1):
        t0 = time.perf_counter()
        M, L, Acc, ids, out = oracle_big_blocks(Q[0, 0], K[0, 0], V[0, 0], [b], difference=THETA)
        dt += time.perf_counter() - t0
        window = G * (G + 1) // 2 + (G * G if b > 0 else 0)
        sample_pairs += window + G * int(ids[b].numel())
        blocks.append(b)
        if dt >= limit_s:
            break
    cap_total = sum(bb * G - 2 * BLOCK for bb in range(1, NB))
    layer_pairs = H * (G * (G + 1) // 2 + (NB - 1) * (G * G + G * (G + 1) // 2) + G * cap_total)
    ms = dt * 1e3 * layer_pairs / sample_pairs
    desc = (f"CPU restatement (torch fp32 matmuls, bf16 rounding points) on {cores} threads: 1 head of the "
            f"{N}-token layer, query rows of big blocks {blocks[0]}..{blocks[-1]} ({len(blocks)} x 2048 rows, "
            f"{sample_pairs / 1e9:.2f} G query-key pairs, {dt:.1f} s), scaled to the layer's "
            f"{layer_pairs / 1e9:.1f} G pairs at density 1")
    return ms, desc, cores


def cpu_config0():
    """The reference-runnable CPU case: one layer at seq 4096, 32 query / 8 KV heads, fp32, no
    RoPE, whole operator through the CPU restatement without rounding (mode "fp32") on all host
    threads; 1 warm-up + 3 timed calls, median.  With a GPU the bf16 CUDA operator runs on the
    same inputs (cast to bf16) and its distance to the fp32 result is reported with its time.
    Prints one JSON line of its own (not the benchmark line)."""
    import torch
    from oracle.anchor_oracle import anchor_attn_oracle, make_inputs
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    N0 = 4096
    Q, K, V = make_inputs(N0, H, HKV, seed=0, rope=False, dtype=torch.float32)
    times = []
    res = None
    for i in range(4):
        t0 = time.perf_counter()
        res = anchor_attn_oracle(Q, K, V, difference=THETA, mode="fp32")
        if i > 0:
            times.append((time.perf_counter() - t0) * 1e3)
    G = BLOCK * STEP
    cap = H * sum(b * G - 2 * BLOCK for b in range(1, N0 // G))
    line = {"config": f"configs[0]: anchor_attn layer, seq {N0}, {H}q/{HKV}kv heads, head_dim {D}, fp32, no RoPE, "
                      f"block {BLOCK}, step {STEP}, theta {THETA}",
            "cpu_ms_median": statistics.median(times), "cpu_ms_runs": times, "cores": cores, "kind": "port",
            "density": float(res.counts.sum()) / cap, "data": "synthetic"}
    if torch.cuda.is_available():
        from anchor_attention_b200 import AnchorAttnCall
        call = AnchorAttnCall(Q.cuda().bfloat16(), K.cuda().bfloat16(), V.cuda().bfloat16(), None, BLOCK, STEP, THETA)
        for _ in range(3):
            call.run()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(10):
            out = call.run()
        ev1.record()
        torch.cuda.synchronize()
        call.check_status()
        err = (out.float().cpu() - res.out).abs()
        line.update({"gpu_bf16_ms": ev0.elapsed_time(ev1) / 10, "gpu_selected_columns": int(call.counts.sum()),
                     "cpu_selected_columns": int(res.counts.sum()),
                     "gpu_bf16_vs_cpu_fp32_max_abs": float(err.max()), "gpu_bf16_vs_cpu_fp32_mean_abs": float(err.mean())})
    print(json.dumps(line), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    desc, cores = "", 0
    for i in range(args.warmup + args.steps):
        ms, desc, cores = cpu_sample(args.seq)
        if i >= args.warmup:
            vals.append(ms)
    v = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "ms", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": v, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"anchor_attn layer, seq {args.seq}, {H}q/{HKV}kv heads, head_dim {D}, "
                               f"block {BLOCK}, step {STEP}, theta {THETA}"},
        "cpu_baseline": {"value": v, "unit": "ms", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from anchor_attention_b200 import AnchorAttnCall, launches_per_forward
    from anchor_attention_b200.parallel import HeadShardedAnchorAttn, PushedOutput, gather_heads, head_partition
    from anchor_attention_b200.synthetic import make_inputs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    W = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if W != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={W}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if W > 1:
        dist.init_process_group("nccl", device_id=dev)
    N = args.seq
    q_lo, q_hi, kv_lo, kv_hi = head_partition(H, HKV, W, rank)
    h = q_hi - q_lo
    THETA = args.theta          # 12 unless the auxiliary sparse-regime run is asked for
    Q, K, V = make_inputs(N, H, HKV, seed=0, rope=True, device=dev, heads=(q_lo, q_hi, kv_lo, kv_hi),
                          q_shift=args.q_shift)
    push = W > 1 and args.exchange == "push"
    exchange_note = ""
    if push:
        # every rank's copy of the assembled [1,N,H,D] output lives in symmetric memory; step 3
        # stores this rank's heads into all copies, a barrier replaces the all-gather
        try:
            pushed = PushedOutput(1, N, H, D, torch.bfloat16, dev)
            failed = 0
        except Exception as e:      # symmetric memory could not be set up on this machine
            failed, exchange_note = 1, f"symmetric memory unavailable ({type(e).__name__}), used the all-gather"
        flag = torch.tensor([failed], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()):
            push = False
            args.exchange = "all_gather"
            exchange_note = exchange_note or "symmetric memory unavailable on another rank, used the all-gather"
    if push:
        out_view = pushed.bufs[0][:, :, q_lo:q_hi].permute(0, 2, 1, 3)
        head_off = q_lo * D * 2
        gathered = None
    else:
        out_local = torch.empty((1, N, h, D), dtype=torch.bfloat16, device=dev)        # token-major
        out_view = out_local.permute(0, 2, 1, 3)
        gathered = torch.empty((W, 1, N, h, D), dtype=torch.bfloat16, device=dev) if W > 1 else None
    call = AnchorAttnCall(Q, K, V, None, BLOCK, STEP, THETA, out=out_view)

    def step(ev=None):
        call.step1()
        call.step2()
        if ev is not None:
            ev[0].record()
        if push:
            _, ptrs, handle = pushed.next()
            call.step3_push([p + head_off for p in ptrs])
        else:
            call.step3()
        if ev is not None:
            ev[1].record()
        if push:
            handle.barrier(channel=0)
        elif W > 1:
            gather_heads(out_local, None, gathered)

    def barrier():
        if W > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    k_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for i in range(args.steps):
        step(k_ev[i])
    t1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = t0.elapsed_time(t1) / args.steps
    k3_ms = statistics.mean(a.elapsed_time(b) for a, b in k_ev)
    counts_total = int(call.counts.sum())

    # ---- end to end through the public entry point, host buffers in, host result out
    from anchor_attention_b200 import anchor_attn_host
    hq, hk, hv = (t.cpu().pin_memory() for t in (Q, K, V))
    hout = torch.empty((1, h, N, D), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(1, min(args.steps, 3))

    sharded = HeadShardedAnchorAttn(None, BLOCK, STEP, THETA, exchange=args.exchange) if W > 1 else None

    def e2e_step():
        if W == 1:
            # host buffers in, host buffer out; the KV-head groups are streamed so that the copies
            # of one group overlap the computation of another
            anchor_attn_host(hq, hk, hv, hout, None, BLOCK, STEP, THETA, device=dev)
            return
        dq, dk, dv = hq.to(dev, non_blocking=True), hk.to(dev, non_blocking=True), hv.to(dev, non_blocking=True)
        full = sharded(dq, dk, dv)                                       # [1,N,H,D] on every rank
        hout.copy_(full[:, :, q_lo:q_hi].permute(0, 2, 1, 3), non_blocking=True)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- max over ranks
    stats = torch.tensor([ms, k3_ms, e2e_ms, float(counts_total)], dtype=torch.float64, device=dev)
    if W > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, k3_ms, e2e_ms = mx[0].item(), mx[1].item(), mx[2].item()
        counts_all = int(sm[3].item())
    else:
        counts_all = counts_total
    if rank == 0:
        peak_tf, peak_gbs, peak_src = measured_peaks()
        f1, f2, f3 = algorithmic_flops(N, H, counts_all)
        G = BLOCK * STEP
        cap = H * sum(b * G - 2 * BLOCK for b in range(1, N // G))
        f3_rank = f3 / W                               # the launch timed on one rank handles 1/W of the heads
        achieved = f3_rank / (k3_ms * 1e-3) / 1e12
        tile_pair_loads = counts_all / W * (G // (2 * BLOCK)) / BLOCK     # ids x 8 query-tile pairs / 128 ids per tile
        ref_n = min(STEP3_DRAM_CAPTURES, key=lambda n: abs(n - N))
        ref_bytes, ref_loads = STEP3_DRAM_CAPTURES[ref_n]
        traffic = ref_bytes * tile_pair_loads / ref_loads
        aux = args.q_shift != 0.0 or args.theta != 12.0
        line = {
            "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": W, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16",
            "data": f"synthetic, AUXILIARY distribution (q_shift {args.q_shift}, theta {args.theta})" if aux else "synthetic",
            "config": {"workload": f"anchor_attn layer, seq {N}, {H}q/{HKV}kv heads, head_dim {D}, block {BLOCK}, "
                                   f"step {STEP}, theta {THETA}",
                       "parallelism": (f"heads by KV group over {W} GPU(s), " +
                                       ("step 3 stores its rows into every rank's output over NVLink, one barrier"
                                        if push else "one NCCL all-gather")) if W > 1 else "single GPU",
                       "exchange_note": exchange_note,
                       "l2": "inputs_exceed_l2", "density": counts_all / cap if cap else 0.0,
                       "selected_columns": counts_all},
            "algorithmic_tflop": {"step1": f1 / 1e12, "step2": f2 / 1e12, "step3": f3 / 1e12},
            "layer_tflops": (f1 + f2 + f3) / (ms * 1e-3) / 1e12,
            "roofline": {"kernel": "step 3 (gathered sparse flash attention)", "bound": "tensor",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "traffic": traffic, "traffic_unit": f"DRAM bytes per launch (ncu capture at {ref_n} tokens, scaled by tile loads)",
                         "peak_source": f"{peak_src} (sustained bf16)", "launch_ms": k3_ms},
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": W * sum(t.numel() * 2 for t in (hq, hk, hv)),
                    "d2h_bytes_per_step": W * hout.numel() * 2, "steps": e2e_steps},
            "gpu_launches": launches_per_forward() * args.steps,
            "clocks": clocks,
        }
        if W == 1 and not args.no_cpu_baseline:
            v, desc, cores = cpu_sample(N)
            line["cpu_baseline"] = {"value": v, "unit": "ms", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if W > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq", type=int, default=131072)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--q-shift", type=float, default=0.0,
                    help="auxiliary distribution: add this to Q before the stripe step (sparse selection); "
                         "not the benchmark configuration")
    ap.add_argument("--theta", type=float, default=THETA, help="auxiliary runs only; the benchmark uses 12")
    ap.add_argument("--exchange", default="push", choices=["push", "all_gather"],
                    help="how the head outputs reach every rank when N > 1")
    ap.add_argument("--cpu-config0", action="store_true",
                    help="auxiliary: time the CPU restatement on the fp32 4096-token case and stop")
    args = ap.parse_args()
    if args.cpu_config0:
        if int(os.environ.get("RANK", "0")) == 0:
            cpu_config0()
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
