#!/usr/bin/env python
"""Benchmark of the INT8 FlashAttention forward hot path.

One "step" = one pass of the hot path over one batch of synthetic input: the fused quantisation
prologue (fp16 Q/K/V -> int8 + scales) followed by the attention forward, on the workload the
headline metric is quoted on (full-int8, batch 4, heads 32, seq 8192, head_dim 128, non-causal,
sm_scale 1/sqrt(128), Q/K/V fp16 ~ N(0,1) from a seed).  With --gpus N (launched under
torch.distributed.run) every rank processes its own batch of that size -- (batch, head) pairs are
independent, so there is no data-path collective -- and the reported value is the work of all
ranks over the slowest rank's time (weak scaling).

Prints ONE JSON line.  `--impl reference` times the reference's CPU math (the oracle port) on a
bounded sample of the same workload on the host cores instead.
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (variant, B, H, N, D, causal, std, outlier)
    "c2_full_b4_h32_n8192_d128": ("full", 4, 32, 8192, 128, False, 1.0, False),
    "c3_half_b8_h32_n4096_d128_causal": ("half", 8, 32, 4096, 128, True, 1.0, True),
    "c4shard_full_b8_h64_n4096_d128": ("full", 8, 64, 4096, 128, False, 1.0, False),
    "c1_full_b1_h4_n512_d64": ("full", 1, 4, 512, 64, False, 1.0, False),
    # the other head dims of the reference's sweep (benchmark.py:23 runs d=64; the ops accept 16 to 256)
    "d64_full_b4_h32_n8192": ("full", 4, 32, 8192, 64, False, 1.0, False),
    "d64_half_b4_h32_n8192_causal": ("half", 4, 32, 8192, 64, True, 1.0, True),
    "d256_full_b4_h16_n8192": ("full", 4, 16, 8192, 256, False, 1.0, False),
    "d256_half_b4_h16_n8192_causal": ("half", 4, 16, 8192, 256, True, 1.0, True),
    # long-context causal ring over all ranks (sequence-parallel; needs --gpus >= 2): N is the GLOBAL sequence
    "c5_ring_full_b1_h32_n131072_d128_causal": ("full", 1, 32, 131072, 128, True, 0.5, False),
    # small cases of the same kernels for profiler captures (a few hundred MB on the device)
    "prof_full_b2_h16_n4096_d128": ("full", 2, 16, 4096, 128, False, 1.0, False),
    "prof_half_b2_h16_n4096_d128_causal": ("half", 2, 16, 4096, 128, True, 1.0, True),
}
DEFAULT_WORKLOAD = "c2_full_b4_h32_n8192_d128"
METRIC = "INT8 attn fwd effective TOPS (4*B*H*N^2*d / t, halved for causal), prologue included"
LAUNCHES_PROLOGUE_FULL = 2      # kernels of the quantisation prologue per step: Q rows + K rows + V column absmax in one grid; V quantise
LAUNCHES_PROLOGUE_HALF = 1      # Q rows + K rows in one grid


def config_of(workload):
    """The `config` object of the JSON line -- the same for this arm and the reference arm."""
    variant, B, H, N, D, causal, std, outlier = WORKLOADS[workload]
    return {"workload": workload, "variant": variant, "B_per_gpu": B, "H": H, "N": N, "D": D, "causal": causal,
            "sm_scale": D ** -0.5, "quantised_in_step": True,
            "l2": "inputs exceed L2 (%.0f MiB of fp16 Q/K/V per step)" % (3 * B * H * N * D * 2 / 2 ** 20),
            "sharding": "batch x heads, no collective"}


def attn_ops(B, H, N, D, causal):
    ops = 4.0 * B * H * N * N * D
    return ops / 2 if causal else ops


def prologue_bytes(B, H, N, D, full):
    """Algorithmic bytes of the quantisation prologue: every input read once, every output written once."""
    E = B * H * N * D
    if full:
        return 3 * E * 2 + 3 * E + (2 * B * H * N + B * H * D) * 4
    return 2 * E * 2 + 2 * E + 2 * B * H * N * 4


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            c = [x.strip() for x in r.split(",")]
            if len(c) < 7:
                continue
            try:
                sm.append(float(c[0]))
                mx.append(float(c[1]))
                power.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def synth(B, H, N, D, std, outlier, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    q, k, v = (std * torch.randn(B, H, N, D, device=device, generator=g, dtype=torch.float32) for _ in range(3))
    if outlier:
        ch = int(torch.randint(0, D, (1,), device=device, generator=g))
        q[..., ch] *= 20
        k[..., ch] *= 20
    return q.half(), k.half(), v.half()


def cpu_reference_leg(workload, budget_s=15.0, max_heads=256):
    """The reference's PyTorch/Triton math restated for CPU (oracle port), timed on whole (batch, head)
    slices of the workload with all host threads; the bounded sample is scaled to the metric's unit."""
    from oracle import intfa_oracle as O
    variant, B, H, N, D, causal, std, outlier = WORKLOADS[workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sm = D ** -0.5
    q, k, v = synth(1, 1, N, D, std, outlier, 4242, "cpu")
    heads, t_total = 0, 0.0
    while heads < max_heads and (heads == 0 or t_total < budget_s):
        t0 = time.perf_counter()
        q8, qs = O.quant_pertoken(q)
        k8, ks = O.quant_pertoken(k)
        if variant == "full":
            v8, vs = O.quant_perchannel(v)
            O.attention_full_int8(q8, k8, v8, qs, ks, vs, causal, sm, G=128 if D >= 128 else 64)
        else:
            O.attention_int8(q8, k8, v, qs, ks, causal, sm, G=128 if D >= 128 else 64)
        t_total += time.perf_counter() - t0
        heads += 1
    tops = attn_ops(1, 1, N, D, causal) * heads / t_total / 1e12
    return {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": "%d of %d (batch,head) slices of %s, %.1f s of CPU work, prologue included"
                      % (heads, B * H, workload, t_total),
            "ms_per_slice": 1e3 * t_total / heads}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    base = cpu_reference_leg(args.workload, budget_s=8.0, max_heads=4)      # warm-up of the host path
    t0 = time.perf_counter()
    vals = [cpu_reference_leg(args.workload, budget_s=4.0, max_heads=2) for _ in range(max(1, min(args.steps, 5)))]
    dt = time.perf_counter() - t0
    value = statistics.mean(v["value"] for v in vals)
    variant, B, H, N, D, causal, std, outlier = WORKLOADS[args.workload]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": 1, "ms_per_step": 1e3 * dt / len(vals), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": config_of(args.workload),
            "note": "each step = a bounded sample of whole (batch,head) slices of the workload on the host cores",
            "cpu_baseline": {"value": value, "unit": "TOPS", "cores": base["cores"], "kind": "port",
                             "sample": vals[0]["sample"]},
            "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def measure_ring(pkg, dist, rank, world, local_rank, dev, workload, steps, warmup, prefetch=None):
    """Long-context causal full-int8 attention, sequence sharded zigzag over the ranks: every rank owns
    half-chunks (rank, 2*world-1-rank) of the global sequence, quantises them (per-channel V absmax
    all-reduced), and runs the ascending ring (int8 K/V + fp32 K scales by NCCL send/recv).  A step =
    prologue + ring forward of the whole sequence; strong scaling (the global problem is fixed).
    Returns (ms per step as the max over ranks, clocks of rank 0 or None, half-chunk rows)."""
    variant, B, H, N, D, causal, std, outlier = WORKLOADS[workload]
    nh = N // (2 * world)
    sm_scale = D ** -0.5
    parts = []
    for c in (rank, 2 * world - 1 - rank):            # each half-chunk from its own seed: independent of world size
        g = torch.Generator(device=dev).manual_seed(5000 + c)
        parts.append([std * torch.randn(B, H, nh, D, device=dev, generator=g, dtype=torch.float32) for _ in range(3)])
    q, k, v = (torch.cat([parts[0][i], parts[1][i]], dim=2).half() for i in range(3))
    del parts

    def step():
        q8, qs = pkg.quant_pertoken(q)
        k8, ks = pkg.quant_pertoken(k)
        v8, vs = pkg.shard.quantize_v_global(v, "per_channel")
        return pkg.shard.ring_attention_causal(q8, k8, v8, qs, ks, vs, sm_scale, variant="full", prefetch=prefetch)

    def barrier():
        dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(dev)

    for _ in range(warmup):
        step()
    pkg.check_status(dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    pkg.check_status(dev)
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), clocks, nh


def ring_self_check(pkg, dist, rank, world, local_rank, dev):
    """Small ring run (2048 tokens per rank) whose local output must equal, bit for bit, the same rows of a
    single-device causal pass over the whole sequence computed on this rank.  Returns "bit-equal" or a
    description of the mismatch, the same on every rank."""
    B, H, D = 1, 4, 128
    N = 2048 * world
    g = torch.Generator(device=dev).manual_seed(777)          # same tensors on every rank
    q, k, v = (0.5 * torch.randn(B, H, N, D, device=dev, generator=g, dtype=torch.float32) for _ in range(3))
    q, k, v = q.half(), k.half(), v.half()
    sp = lambda t: pkg.shard.zigzag_split(t, world, rank).contiguous()
    q8, qs = pkg.quant_pertoken(sp(q))
    k8, ks = pkg.quant_pertoken(sp(k))
    v8, vs = pkg.shard.quantize_v_global(sp(v), "per_channel")
    loc = pkg.shard.ring_attention_causal(q8, k8, v8, qs, ks, vs, 0.09, variant="full")
    fq8, fqs = pkg.quant_pertoken(q)
    fk8, fks = pkg.quant_pertoken(k)
    fv8, fvs = pkg.quant_perchannel(v)
    one = pkg.attention_full_int8(fq8, fk8, fv8, fqs, fks, fvs, True, 0.09)
    pkg.check_status(dev)
    want = sp(one)
    bad = torch.tensor([0 if torch.equal(loc, want) else 1, 0 if torch.equal(v8, sp(fv8)) else 1], device=dev, dtype=torch.int32)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if int(bad[0]) == 0 and int(bad[1]) == 0:
        return "bit-equal"
    return "MISMATCH (output %d, sharded V quantisation %d)" % (int(bad[0]), int(bad[1]))


def measure_c4_strong(pkg, dist, rank, world, local_rank, dev, steps, warmup):
    """Full-int8 B64 H64 N4096 d128 non-causal, the (batch, head) pairs split evenly over the ranks
    (shard.bh_slice), no collective: strong scaling of a fixed global problem.  Returns ms per step (max over ranks)."""
    B, H, N, D = 64, 64, 4096, 128
    dim, s0, s1 = pkg.shard.bh_slice(B, H, world, rank)
    Bl, Hl = (s1 - s0, H) if dim == 0 else (1, s1 - s0)
    q, k, v = synth(Bl, Hl, N, D, 1.0, False, 3000 + rank, dev)
    sm_scale = D ** -0.5

    def step():
        return pkg.int_flash_attention(q, k, v, False, sm_scale, variant="full")

    for _ in range(warmup):
        step()
    pkg.check_status(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(device_ids=[local_rank])
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    dist.barrier(device_ids=[local_rank])
    torch.cuda.synchronize(dev)
    pkg.check_status(dev)
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def int8_peak_tops(peaks):
    """Denominator of the tensor roofline: the int8 GEMM rate measured on this pool (profiles/roofline_inputs.json,
    from `--workload int8_peak`), else twice the measured bf16 burst rate."""
    pj = os.path.join(ROOT, "profiles", "roofline_inputs.json")
    try:
        m = json.load(open(pj)).get("int8_peak", {})
        if m.get("burst_tops"):
            # the attention kernel is timed per launch inside a region of a fraction of a second, at full clocks:
            # the burst figure is the like-for-like denominator
            return float(m["burst_tops"]), "library int8 GEMM (torch._int_mm 8192^3, burst) measured on this pool"
    except Exception:
        pass
    return 2.0 * peaks["bf16_tflops"], "2 x MEASURED_PEAKS.bf16_tflops (burst; int8 dense rate = 2x bf16)"


def run_int8_peak(dev):
    """Library int8 GEMM rate (torch._int_mm, cuBLASLt): burst = best of 10 single calls, sustained = a 3 s loop.
    Only a yardstick for the roofline denominator; no product path calls it."""
    n = 8192
    a = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
    b = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
    for _ in range(5):
        torch._int_mm(a, b)
    torch.cuda.synchronize(dev)
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize(dev)
        best = min(best, e0.elapsed_time(e1))
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    reps, total_ms, calls = 50, 0.0, 0
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < 3.0:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize(dev)
        total_ms += e0.elapsed_time(e1)
        calls += reps
    clocks = sampler.stop()
    ops = 2.0 * n ** 3
    print(json.dumps({"workload": "int8_peak", "how": "torch._int_mm 8192^3 (library kernel, not part of any product path)",
                      "burst_tops": ops / (best * 1e-3) / 1e12, "sustained_tops": ops * calls / (total_ms * 1e-3) / 1e12,
                      "clocks": clocks}), flush=True)


def run_ring(args, pkg, dist, rank, world, local_rank, dev):
    variant, B, H, N, D, causal, std, outlier = WORKLOADS[args.workload]
    if world < 2:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unavailable": "the ring workload needs --gpus >= 2"}), flush=True)
        return
    steps = min(args.steps, 10)
    ms, clocks, nh = measure_ring(pkg, dist, rank, world, local_rank, dev, args.workload, steps, args.warmup,
                                  prefetch=args.ring_prefetch or None)
    check = ring_self_check(pkg, dist, rank, world, local_rank, dev)
    ops = attn_ops(B, H, N, D, True)
    if rank == 0:
        peaks, src = measured_peaks()
        peak, peak_src = int8_peak_tops(peaks)
        value = ops / (ms * 1e-3) / 1e12
        kv_bytes = B * H * nh * (2 * D + 4)           # one int8 K + V half-chunk and its fp32 K scales
        line = {"metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": steps, "warmup": args.warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8",
                "data": "synthetic",
                "config": {"workload": args.workload, "variant": variant, "B": B, "H": H, "N_global": N, "D": D,
                           "causal": True, "layout": "zigzag half-chunks, ascending ring, NCCL send/recv",
                           "half_chunk_rows": nh, "bytes_per_half_chunk_transfer": kv_bytes,
                           "prefetch": args.ring_prefetch or "all transfers posted up front",
                           "l2": "inputs exceed L2"},
                "clocks": clocks, "gpu_launches": steps * (5 + 2 * world + 1), "ring_check": check,
                "roofline": {"bound": "tensor", "kernel": "intfa_fwd_pipe_kernel", "achieved": value / world,
                             "peak": peak, "unit": "TFLOP/s", "frac": value / world / peak, "traffic": None,
                             "peak_source": "per GPU; " + peak_src},
                "e2e": None, "cpu_baseline": None}
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + ["int8_peak"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ring-prefetch", type=int, default=0, help="ring workload: half-chunk transfers posted ahead of the attention launches (0 = all up front)")
    ap.add_argument("--no-multi", action="store_true", help="with --gpus >= 2: skip the ring and strong-scaling sub-measurements")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    pkg = importlib.import_module("int-flashattention_b200")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.workload == "int8_peak":
        if rank == 0:
            run_int8_peak(dev)
        if world > 1:
            dist.destroy_process_group()
        return
    variant, B, H, N, D, causal, std, outlier = WORKLOADS[args.workload]
    full = variant == "full"
    sm_scale = D ** -0.5
    if "ring" in args.workload:
        run_ring(args, pkg, dist, rank, world, local_rank, dev)
        if world > 1:
            dist.destroy_process_group()
        return
    q, k, v = synth(B, H, N, D, std, outlier, 1000 + rank, dev)

    def step():
        return pkg.int_flash_attention(q, k, v, causal, sm_scale, variant=variant)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        o = step()
    pkg.check_status(dev)

    # ---- device-timed region: K steps, plus per-step events around the attention launch alone
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    a1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    ev0.record()
    for i in range(args.steps):
        if full:
            q8, qs, k8, ks, v8, vs = pkg.quant_qkv(q, k, v)
            a0[i].record()
            o = pkg.attention_full_int8(q8, k8, v8, qs, ks, vs, causal, sm_scale)
        else:
            q8, qs, k8, ks = pkg.quant_qkv(q, k)
            a0[i].record()
            o = pkg.attention_int8(q8, k8, v, qs, ks, causal, sm_scale)
        a1[i].record()
    ev1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    attn_ms = statistics.mean(x.elapsed_time(y) for x, y in zip(a0, a1))
    pkg.check_status(dev)
    t = torch.tensor([ms_total, attn_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, attn_ms = float(t[0]), float(t[1])
    ms_per_step = ms_total / args.steps
    ops_step = attn_ops(B, H, N, D, causal)
    value = ops_step * world / (ms_per_step * 1e-3) / 1e12
    launches_per_step = (LAUNCHES_PROLOGUE_FULL if full else LAUNCHES_PROLOGUE_HALF) + 1      # prologue + attention

    # ---- end-to-end through the public API with HOST buffers (pinned): H2D of q,k,v and D2H of o every step
    e2e = None
    if not args.no_e2e:
        # two sets of pinned host inputs/outputs (alternating), so that no step reuses a buffer still in flight
        hq, hk, hv = (x.cpu().pin_memory() for x in (q, k, v))
        hin = [(hq, hk, hv), tuple(t.clone().pin_memory() for t in (hq, hk, hv))]
        hout = [torch.empty((B, H, N, D), dtype=torch.float16).pin_memory() for _ in range(2)]
        n_e2e = max(3, min(args.steps, 10))

        # (i) one call after the other on one stream: copy in, prologue + attention, copy out
        dq, dk, dv = (torch.empty_like(x) for x in (q, k, v))

        def serial_step(i):
            a, b_, c = hin[i & 1]
            dq.copy_(a, non_blocking=True)
            dk.copy_(b_, non_blocking=True)
            dv.copy_(c, non_blocking=True)
            out = pkg.int_flash_attention(dq, dk, dv, causal, sm_scale, variant=variant)
            hout[i & 1].copy_(out, non_blocking=True)

        for i in range(2):
            serial_step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_e2e):
            serial_step(i)
        e1.record()
        barrier()
        t_serial = e0.elapsed_time(e1) / n_e2e
        del dq, dk, dv

        # (ii) the same calls through HostPipeline (the package's API for host-resident tensors): every step's
        # H2D copies, kernels and D2H copy are issued inside the timed region, on three streams, so that the copies of
        # neighbouring steps overlap the kernels
        pipe = pkg.HostPipeline((B, H, N, D), dev, causal=causal, sm_scale=sm_scale, variant=variant, depth=2)
        for i in range(2):
            pipe.submit(*hin[i & 1], hout[i & 1])
        pipe.synchronize()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(pipe.s_in)
        for i in range(n_e2e):
            last = pipe.submit(*hin[i & 1], hout[i & 1])
        e1.record(pipe.s_out)                      # after the last D2H copy, the last thing to finish
        pipe.synchronize()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1) / n_e2e, t_serial], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": ops_step * world / (float(te[0]) * 1e-3) / 1e12, "unit": "TOPS",
               "ms_per_step": float(te[0]), "steps": n_e2e,
               "h2d_bytes_per_step": 3 * q.numel() * 2, "d2h_bytes_per_step": hout[0].numel() * 2,
               "how": "HostPipeline: pinned host buffers, copy-in / compute / copy-out streams, 2 buffer sets",
               "serial_value": ops_step * world / (float(te[1]) * 1e-3) / 1e12, "serial_ms_per_step": float(te[1])}
        del hq, hk, hv, hin, hout, pipe

    # ---- with 2 or more GPUs, and on the default workload: the two multi-GPU decompositions as sub-objects of the line
    multi = {}
    if world > 1 and args.workload == DEFAULT_WORKLOAD and not args.no_multi:
        del q, k, v, o
        torch.cuda.empty_cache()
        rw = "c5_ring_full_b1_h32_n131072_d128_causal"
        r_ms, _, r_nh = measure_ring(pkg, dist, rank, world, local_rank, dev, rw, steps=4, warmup=2)
        torch.cuda.empty_cache()
        multi["ring_check"] = ring_self_check(pkg, dist, rank, world, local_rank, dev)
        c4_ms = measure_c4_strong(pkg, dist, rank, world, local_rank, dev, steps=3, warmup=1)
        torch.cuda.empty_cache()
        r_ops = attn_ops(1, 32, 131072, 128, True)
        c4_ops = attn_ops(64, 64, 4096, 128, False)
        multi["ring"] = {"workload": rw, "value": r_ops / (r_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": r_ms,
                         "per_gpu": r_ops / (r_ms * 1e-3) / 1e12 / world, "scaling": "strong", "half_chunk_rows": r_nh,
                         "transport": "NCCL send/recv of int8 K/V + fp32 K scales into local HBM, all transfers posted up front"}
        multi["c4_strong"] = {"workload": "full-int8 B64 H64 N4096 d128 non-causal, (batch, head) pairs split over the ranks",
                              "value": c4_ops / (c4_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": c4_ms,
                              "per_gpu": c4_ops / (c4_ms * 1e-3) / 1e12 / world, "scaling": "strong", "collective": "none"}

    if rank == 0:
        peaks, src = measured_peaks()
        peak_int8, peak_src = int8_peak_tops(peaks)
        for kname in ("ring", "c4_strong"):
            if kname in multi:
                multi[kname]["frac"] = multi[kname]["per_gpu"] / peak_int8
        achieved = ops_step / (attn_ms * 1e-3) / 1e12
        prof = {}
        pj = os.path.join(ROOT, "profiles", "roofline_inputs.json")
        if os.path.exists(pj):
            prof = json.load(open(pj)).get(args.workload, {})
        roofline = {"bound": "tensor", "kernel": "intfa_fwd_pipe_kernel",
                    "achieved": achieved, "peak": peak_int8,
                    "unit": "TFLOP/s", "frac": achieved / peak_int8,
                    "frac_of_2x_bf16_burst": achieved / (2.0 * peaks["bf16_tflops"]),
                    "frac_of_2x_bf16_sustained": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                    "traffic": prof.get("attn_dram_bytes_per_launch"),
                    "traffic_source": "constant from an earlier one-pass ncu capture of this launch (profiles/), not measured by this run",
                    "peak_source": peak_src + " (MEASURED_PEAKS: %s)" % src,
                    "kernel_ms": attn_ms,
                    "prologue": {"bound": "hbm", "ms": ms_per_step - attn_ms,
                                 "achieved": prologue_bytes(B, H, N, D, full) / ((ms_per_step - attn_ms) * 1e-3) / 1e9,
                                 "peak": peaks["hbm_gbs"], "unit": "GB/s"}}
        roofline["prologue"]["frac"] = roofline["prologue"]["achieved"] / peaks["hbm_gbs"]
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_reference_leg(args.workload)
        line = {"metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "s8", "data": "synthetic",
                "config": config_of(args.workload),
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
                "roofline": roofline, "cpu_baseline": cpu,
                "pct_of_nominal_int8_peak": 100.0 * achieved / 4500.0}
        line.update(multi)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
