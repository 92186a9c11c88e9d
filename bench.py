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

``--triton-bar --ref-root <checkout of the reference>`` is an optional leg of its
own: it runs the reference's unmodified ``anchor_attn_test_time``
(anchor_attn/src/ops/anchor_attn_v4.py:328-354, Triton kernels compiled on the
spot) on the same inputs with CUDA events and prints one JSON line with its
times next to this library's on the same GPU.  Nothing else in this file, and
nothing in the package, imports the reference.

Besides the timing the line carries ``parity`` (sampled (head, big block) pairs of
the timed run's own output and id lists against the CPU oracle, outside the timed
region), ``aux_sparse`` (step 3 on the labelled auxiliary distribution, where the
id lists are sparse) and ``clock_normalised`` (step-3 cycles per key/value tile at
two sequence lengths from the sampled SM clock).
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
# GPU, from single-pass ncu captures of this benchmark (profiles/launch_list_seq131072.md): sequence
# length -> (bytes, K/V tile-pair loads of 64 KB by all CTAs).  Other sizes, densities and per-rank
# shares are scaled from the nearest entry by their tile-pair loads.
STEP3_DRAM_CAPTURES = {32768: (1.205e9, 483840), 131072: (7.583e9, 8225280)}


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


def workload_config(N, W, exchange, theta=THETA, note=""):
    """The ``config`` object of the JSON line; both arms print the same one."""
    if W > 1:
        par = f"heads by KV group over {W} GPU(s), " + (
            "step 3 stores its rows into every rank's output over NVLink, one barrier" if exchange == "push"
            else "one NCCL all-gather")
    else:
        par = "single GPU"
    return {"workload": f"anchor_attn layer, seq {N}, {H}q/{HKV}kv heads, head_dim {D}, block {BLOCK}, "
                        f"step {STEP}, theta {theta}",
            "parallelism": par, "exchange_note": note, "l2": "inputs_exceed_l2"}


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


def cpu_config0(with_gpu=True):
    """The reference-runnable CPU case: one layer at seq 4096, 32 query / 8 KV heads, fp32, no
    RoPE, whole operator through the CPU restatement without rounding (mode "fp32") on all host
    threads; 1 warm-up + 3 timed calls, median (measured, nothing extrapolated).  With a GPU
    the bf16 CUDA operator runs on the same inputs (cast to bf16) and its distance to the fp32
    result is reported with its time.  Returns the record."""
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
    if with_gpu and torch.cuda.is_available():
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
    return line


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    desc, cores = "", 0
    # every step is a bounded sample; the whole run stays within a few minutes
    limit_s = max(2.0, min(12.0, 150.0 / (args.warmup + args.steps)))
    for i in range(args.warmup + args.steps):
        ms, desc, cores = cpu_sample(args.seq, limit_s=limit_s)
        if i >= args.warmup:
            vals.append(ms)
    v = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "ms", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": v, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.seq, args.gpus, args.exchange),
        "cpu_baseline": {"value": v, "unit": "ms", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def parity_check(call, Q, K, V, full, N, W, rank, q_lo, theta, dev):
    """Outside the timed region: the run's own output and id lists against the CPU oracle on
    sampled (head, big block) pairs -- heads {0, H-1} x big blocks {1, NB/2, NB-1}.  Head 0 is
    checked by rank 0 and head H-1 by the last rank (which own them and hold their id lists);
    the oracle's output rows are then broadcast and EVERY rank compares its copy of the
    assembled output ``full`` [1,N,H,D] with them, so at N > 1 the rows a rank received from a
    peer are checked as well.  Also compares a per-head checksum of all ranks' copies.
    Returns the ``parity`` object of the JSON line (identical on every rank)."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle.anchor_oracle import oracle_big_blocks
    from parity_util import OUT_MAX_ABS, OUT_MEAN_ABS, check_id_set
    G = BLOCK * STEP
    NB = N // G
    blocks = sorted({min(1, NB - 1), NB // 2, NB - 1})
    checkers = {0: 0, H - 1: W - 1}                      # head -> rank that runs the oracle for it
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // (2 if W > 1 else 1)))
    rows = {}
    sym_diff = selected = band = 0
    ids_ok = True
    t0 = time.perf_counter()
    for head, owner in checkers.items():
        if owner != rank:
            continue
        hl = head - q_lo
        q, k, v = Q[0, hl].cpu(), K[0, hl // (H // HKV)].cpu(), V[0, hl // (H // HKV)].cpu()
        ref = torch.empty((len(blocks), G, D), dtype=torch.float32)
        counts = call.counts.cpu()
        for i, b in enumerate(blocks):
            M, L, Acc, oids, oout = oracle_big_blocks(q, k, v, [b], difference=theta)
            ref[i] = oout[b * G:(b + 1) * G]
            c = int(counts[0, hl, b])
            off = call.id_row_offset(b)
            ids = call.ids[0, hl, off:off + c].cpu()
            selected += c
            sym_diff += len(set(ids.tolist()) ^ set(oids[b].tolist()))
            if b:
                try:
                    band += check_id_set(ids, q, k, torch.nan_to_num(M), D ** -0.5, theta, b, BLOCK, STEP)[0]
                except AssertionError:
                    ids_ok = False
        rows[head] = ref.to(dev)
    out_max = out_mean = 0.0
    for head, owner in checkers.items():
        ref = rows.get(head)
        if ref is None:
            ref = torch.empty((len(blocks), G, D), dtype=torch.float32, device=dev)
        if W > 1:
            dist.broadcast(ref, src=owner)
        for i, b in enumerate(blocks):
            err = (full[0, b * G:(b + 1) * G, head].float() - ref[i]).abs()
            out_max = max(out_max, float(err.max()))
            out_mean = max(out_mean, float(err.mean()))
    # every rank's copy of the assembled output holds the same bits
    sums = torch.stack([full[0, :, h].contiguous().view(torch.int16).to(torch.int64).sum() for h in range(H)])
    stats = torch.tensor([out_max, out_mean, float(sym_diff), float(selected), float(band), 0.0 if ids_ok else 1.0],
                         dtype=torch.float64, device=dev)
    copies_equal = True
    if W > 1:
        hi, lo = sums.clone(), sums.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        copies_equal = bool(torch.equal(hi, lo))
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        stats = torch.stack([mx[0], mx[1], sm[2], sm[3], sm[4], mx[5]])
    out_max, out_mean = stats[0].item(), stats[1].item()
    ok = out_max <= OUT_MAX_ABS and out_mean <= OUT_MEAN_ABS and stats[5].item() == 0.0 and copies_equal
    return {"pairs": [[h, b] for h in checkers for b in blocks], "rows_checked_on": f"all {W} rank(s)",
            "selected": int(stats[3].item()), "sym_diff": int(stats[2].item()), "tie_band": int(stats[4].item()),
            "ids_within_tie_band": stats[5].item() == 0.0, "out_max": out_max, "out_mean": out_mean,
            "tolerance": {"out_max": OUT_MAX_ABS, "out_mean": OUT_MEAN_ABS}, "copies_equal": copies_equal,
            "oracle_s": time.perf_counter() - t0, "ok": bool(ok)}


def timed_steps(call, seconds, sampler_index):
    """Repeats the whole operator for about ``seconds`` with the SM clock sampled, the three steps
    bracketed by CUDA events.  Returns ([step-1, step-2, step-3 ms] medians, median SM MHz)."""
    import torch
    for _ in range(3):
        call.run()
    torch.cuda.synchronize()
    sampler = ClockSampler(sampler_index)
    sampler.start()
    evs = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end:
        for _ in range(4):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record(); call.step1(); e[1].record(); call.step2(); e[2].record(); call.step3(); e[3].record()
            evs.append(e)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    return [statistics.median(e[i].elapsed_time(e[i + 1]) for e in evs) for i in range(3)], clocks.get("sm_mhz")


def aux_measurements(dev, local, main_step3_ms, main_mhz, main_counts, N):
    """Single-GPU extras, outside the headline timing.
    aux_sparse: the labelled AUXILIARY distribution (q_shift 0.5) at 32768 tokens, where the id
    lists are sparse and step 3 runs through its gather pass: density, step times (step 3 with its
    gather pass) and TFLOP/s on the selected pairs for theta 8, 9 and 10, each from a loop of about
    one second with the SM clock sampled; and the same distribution at the benchmark's own length
    for theta 10 (two-second loop).
    clock_normalised: step-3 SM cycles per 128-id tile and query-tile pair (launch time x median
    sampled SM clock / tile pairs / 148 SMs) for the benchmark launch and for the dense
    32768-token layer, each from a loop of about two seconds; equal cycles mean the difference in
    TFLOP/s between the two sizes is the clock under the power cap."""
    import torch
    from anchor_attention_b200 import AnchorAttnCall
    from anchor_attention_b200.synthetic import make_inputs
    N_AUX = 32768
    G = BLOCK * STEP
    cap = H * sum(b * G - 2 * BLOCK for b in range(1, N_AUX // G))
    aux = {"note": "AUXILIARY distribution, not the benchmark configuration", "seq": N_AUX, "q_shift": 0.5, "cases": []}
    Q, K, V = make_inputs(N_AUX, H, HKV, seed=0, rope=True, device=dev, q_shift=0.5)
    for theta in (8.0, 9.0, 10.0):
        call = AnchorAttnCall(Q, K, V, None, BLOCK, STEP, theta)
        t, mhz = timed_steps(call, 1.0, local)
        call.check_status()
        cnt = int(call.counts.sum())
        aux["cases"].append({"theta": theta, "density": cnt / cap, "step1_ms": t[0], "step2_ms": t[1], "step3_ms": t[2],
                             "sm_mhz": mhz, "gathered_tiles": call.gather_slots_used,
                             "step3_tflops_selected_pairs": 4 * D * G * cnt / (t[2] * 1e-3) / 1e12})
    del Q, K, V
    if N > N_AUX:
        # the same distribution at the benchmark's length, theta 10: lists that outgrow the capped gather
        # scratch, so step 3 goes KV head by KV head (plan word 1)
        Q, K, V = make_inputs(N, H, HKV, seed=0, rope=True, device=dev, q_shift=0.5)
        call = AnchorAttnCall(Q, K, V, None, BLOCK, STEP, 10.0)
        t, mhz = timed_steps(call, 2.0, local)
        call.check_status()
        cnt = int(call.counts.sum())
        capN = H * sum(b * G - 2 * BLOCK for b in range(1, N // G))
        aux["at_benchmark_length"] = {
            "seq": N, "theta": 10.0, "density": cnt / capN, "step1_ms": t[0], "step2_ms": t[1], "step3_ms": t[2],
            "sm_mhz": mhz, "step3_in_parts": int(call._view(call.layout.status_off, 5, torch.int32)[4]),
            "launches": call.launches, "step3_tflops_selected_pairs": 4 * D * G * cnt / (t[2] * 1e-3) / 1e12}
        del Q, K, V, call
    Q, K, V = make_inputs(N_AUX, H, HKV, seed=0, rope=True, device=dev)
    call = AnchorAttnCall(Q, K, V, None, BLOCK, STEP, THETA)
    t32, mhz32 = timed_steps(call, 2.0, local)
    ms32 = t32[2]
    cnt32 = int(call.counts.sum())

    def cycles(ms, mhz, cnt):
        pairs = cnt / BLOCK * (G // (2 * BLOCK))          # (128-id tile, 256-row query pair) products
        return ms * 1e-3 * mhz * 1e6 * 148 / pairs if mhz else None

    norm = {"note": "step-3 SM cycles per (128-id tile x 256 query rows), from launch time x median sampled SM clock",
            f"seq{N}": {"step3_ms": main_step3_ms, "sm_mhz": main_mhz, "cycles_per_tile_pair": cycles(main_step3_ms, main_mhz, main_counts),
                        "tflops": 4 * D * G * main_counts / (main_step3_ms * 1e-3) / 1e12},
            f"seq{N_AUX}": {"step3_ms": ms32, "sm_mhz": mhz32, "cycles_per_tile_pair": cycles(ms32, mhz32, cnt32),
                            "tflops": 4 * D * G * cnt32 / (ms32 * 1e-3) / 1e12}}
    return aux, norm


def run_ours(args):
    import torch
    import torch.distributed as dist
    from anchor_attention_b200 import AnchorAttnCall
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
        # stores this rank's heads into all copies, a flag barrier replaces the all-gather
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
    last = {}

    def step(ev=None):
        call.step1()
        call.step2()
        if ev is not None:
            ev[0].record()
        if push:
            buf, ptrs = pushed.next()
            call.step3_push([p + head_off for p in ptrs])
        else:
            call.step3()
        if ev is not None:
            ev[1].record()
        if push:
            pushed.barrier()
            last["full"] = buf
        elif W > 1:
            last["full"] = gather_heads(out_local, None, gathered)
        else:
            last["full"] = out_local

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
    # no bounded device-side wait gave up during the timed loop (synchronises); a failure is reported
    # in the line, it does not stop the run
    device_status = "ok"
    try:
        call.check_status()
        if push:
            pushed.check_status()
    except RuntimeError as e:
        device_status = f"FAILED: {e}"
    parity = None
    if not args.no_parity:
        parity = parity_check(call, Q, K, V, last["full"], N, W, rank, q_lo, THETA, dev)

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
        else:
            # each rank streams its heads through the device (copies overlap the computation of
            # the previous head); every rank ends with the assembled output on the device and
            # its own heads' result back in host memory
            sharded.host_call(hq, hk, hv, hout)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    # the end-to-end result equals the device-resident result bit for bit
    e2e_equal = bool(torch.equal(hout.to(dev).permute(0, 2, 1, 3), last["full"][:, :, q_lo:q_hi]))

    # ---- max over ranks
    stats = torch.tensor([ms, k3_ms, e2e_ms, float(counts_total), 0.0 if e2e_equal else 1.0,
                          0.0 if device_status == "ok" else 1.0], dtype=torch.float64, device=dev)
    if W > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, k3_ms, e2e_ms = mx[0].item(), mx[1].item(), mx[2].item()
        counts_all = int(sm[3].item())
        e2e_equal = mx[4].item() == 0.0
        if mx[5].item() != 0.0 and device_status == "ok":
            device_status = "FAILED on another rank"
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
            "config": workload_config(N, W, args.exchange, THETA, exchange_note),
            "selection": {"density": counts_all / cap if cap else 0.0, "selected_columns": counts_all},
            "algorithmic_tflop": {"step1": f1 / 1e12, "step2": f2 / 1e12, "step3": f3 / 1e12},
            "layer_tflops": (f1 + f2 + f3) / (ms * 1e-3) / 1e12,
            "roofline": {"kernel": "step 3 (gathered sparse flash attention)", "bound": "tensor",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "traffic": traffic, "traffic_unit": f"DRAM bytes per launch (ncu capture at {ref_n} tokens, scaled by tile loads)",
                         "peak_source": f"{peak_src} (sustained bf16)", "launch_ms": k3_ms},
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": W * sum(t.numel() * 2 for t in (hq, hk, hv)),
                    "d2h_bytes_per_step": W * hout.numel() * 2, "steps": e2e_steps, "equals_device_result": e2e_equal},
            # this rank's kernels of the library in the timed region: the operator's own (step 3 enqueues both
            # of its sequences when the gather scratch has no slot for every possible tile; the kernels of the
            # one the device does not choose leave at once) plus, head-parallel, the flag barrier
            "gpu_launches": (call.launches + (1 if push else 0)) * args.steps,
            "device_status": device_status,
            "clocks": clocks,
        }
        if parity is not None:
            line["parity"] = parity
        if W == 1 and not args.no_aux:
            del hq, hk, hv, hout
            line["aux_sparse"], line["clock_normalised"] = aux_measurements(
                dev, local, k3_ms, clocks.get("sm_mhz") if clocks else None, counts_all, N)
        if W == 1 and not args.no_cpu_baseline:
            v, desc, cores = cpu_sample(N)
            line["cpu_baseline"] = {"value": v, "unit": "ms", "cores": cores, "kind": "port", "sample": desc}
            c0 = cpu_config0(with_gpu=False)
            line["cpu_baseline"]["config0_ms"] = c0["cpu_ms_median"]
            line["cpu_baseline"]["config0"] = (c0["config"] + f"; measured, not extrapolated: median of 3 calls on "
                                               f"{c0['cores']} threads")
        print(json.dumps(line), flush=True)
    if W > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------
# The reference's own kernels on this GPU (optional leg)
# --------------------------------------------------------------------------
def run_triton_bar(args):
    """Times the reference's unmodified ``anchor_attn_test_time`` (anchor_attn/src/ops/
    anchor_attn_v4.py:328-354: search = steps 1 + 2, compute = step 3; Triton kernels compiled
    for this GPU) and this library on the same inputs: 3 warm-up calls, then CUDA events around
    ``--steps`` calls, median.  K and V are expanded to the query head count for the reference,
    as its caller does (modules/llama/anchor_attention.py:89-91).  Prints one JSON line."""
    import importlib
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    theta = args.theta
    line = {"leg": "triton_bar", "seq": args.seq, "heads": f"{H}q/{HKV}kv", "theta": theta}
    if args.q_shift != 0.0 or theta != THETA:
        line["data"] = f"synthetic, AUXILIARY distribution (q_shift {args.q_shift}, theta {theta})"
    root = args.ref_root
    if not root or not os.path.isdir(root):
        line["triton_bar"] = f"unavailable: no reference checkout at {root!r} (pass --ref-root)"
        print(json.dumps(line), flush=True)
        return
    try:
        sys.path.insert(0, os.path.abspath(root))
        ref = importlib.import_module("anchor_attn.src.ops.anchor_attn_v4")
    except Exception as e:      # import of the reference (or of Triton) failed
        line["triton_bar"] = f"unavailable: {type(e).__name__}: {e}"
        print(json.dumps(line), flush=True)
        return
    from anchor_attention_b200 import AnchorAttnCall
    from anchor_attention_b200.synthetic import make_inputs
    dev = torch.device("cuda", 0)
    N = args.seq
    Q, K, V = make_inputs(N, H, HKV, seed=0, rope=True, device=dev, q_shift=args.q_shift)
    Ke, Ve = (t.repeat_interleave(H // HKV, dim=1).contiguous() for t in (K, V))

    def ev():
        return torch.cuda.Event(enable_timing=True)

    full, search, compute = [], [], []
    out_ref = None
    for i in range(3 + args.steps):
        a, b = ev(), ev()
        a.record()
        out_ref, ratio, s_ms, c_ms = ref.anchor_attn_test_time(Q, Ke, Ve, None, BLOCK, STEP, theta, True)
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            full.append(a.elapsed_time(b)); search.append(s_ms); compute.append(c_ms)
    del Ke, Ve
    call = AnchorAttnCall(Q, K, V, None, BLOCK, STEP, theta)
    ours = []
    for i in range(3 + args.steps):
        a, b = ev(), ev()
        a.record()
        out = call.run()
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            ours.append(a.elapsed_time(b))
    err = (out.float() - out_ref.float()).abs()
    line["triton_bar"] = {"ms": statistics.median(full), "step12_ms": statistics.median(search),
                          "step3_ms": statistics.median(compute), "sparsity_ratio": float(ratio),
                          "timing": "ms: CUDA events around anchor_attn_test_time; step12/step3: its own wall clocks"}
    line["ours_ms"] = statistics.median(ours)
    line["speedup"] = statistics.median(full) / statistics.median(ours)
    line["out_max_abs_diff"], line["out_mean_abs_diff"] = float(err.max()), float(err.mean())
    print(json.dumps(line), flush=True)


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
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the run's own output")
    ap.add_argument("--no-aux", action="store_true", help="skip the auxiliary sparse-regime and clock-normalised runs")
    ap.add_argument("--triton-bar", action="store_true",
                    help="optional leg: time the reference's own Triton kernels from --ref-root on this GPU and stop")
    ap.add_argument("--ref-root", default=None, help="checkout of the reference project (for --triton-bar only)")
    args = ap.parse_args()
    if args.triton_bar:
        run_triton_bar(args)
        return
    if args.cpu_config0:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(cpu_config0()), flush=True)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
