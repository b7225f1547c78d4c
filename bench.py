"""Benchmark of the async-TP hot path on B200: fused all-gather->matmul + matmul->reduce-scatter.

    python bench.py --gpus N --steps K --warmup W            # this repository's kernels
    python bench.py --impl reference --gpus N ...            # the reference's unfused CPU path

Workload (BASELINE config 2, Llama-3-8B MLP at TP 8, bf16): 32768 tokens x hidden 4096 sharded
along the sequence over the N ranks; every rank holds the TP-8 weight slices w1, w3 [4096,1792]
and w2 [1792,4096] whatever N is, so the work per GPU is fixed (weak scaling). One step =
fused_all_gather_matmul(x_shard, [w1, w3]) followed by fused_matmul_reduce_scatter(h, w2) with
h = silu(h1) * h3 [32768,1792]. Synthetic data: activations ~N(0,1) seeded by rank, weights
~N(0,0.02). Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TOKENS, HIDDEN, FFN_PER_RANK = 32768, 4096, 1792
FLOPS_AG = FLOPS_RS = FLOPS_STEP = 0.0


def _set_tokens(tokens: int) -> None:
    """--tokens shrinks the workload (ncu captures); the default is the BASELINE size."""
    global TOKENS, FLOPS_AG, FLOPS_RS, FLOPS_STEP
    TOKENS = tokens
    FLOPS_AG = 2.0 * TOKENS * HIDDEN * (2 * FFN_PER_RANK)   # per GPU, w1 and w3
    FLOPS_RS = 2.0 * TOKENS * FFN_PER_RANK * HIDDEN         # per GPU, w2
    FLOPS_STEP = FLOPS_AG + FLOPS_RS


_set_tokens(TOKENS)
NOMINAL_BF16 = 2.25e15      # dense bf16 peak named by the task
NVLINK_BPS = 900e9          # per direction per GPU, nominal
METRIC = "AG+GEMM / GEMM+RS TFLOP/s (whole job; per-GPU and % of roofline beside it)"
CPU_SAMPLE_TOKENS = 4096    # the CPU arms run this many of the 32768 tokens per step


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("bf16_tflops_sustained") or d.get("bf16_tflops"), "measured"
    return 1400.0, "fallback"


_SAMPLER_CHILD = r"""
import sys, time
import pynvml
pynvml.nvmlInit()
h = pynvml.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
print("max", pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM), flush=True)
while True:
    try:
        bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
    except AttributeError:
        bits = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
    print(time.time_ns(), pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), int(bits), flush=True)
    time.sleep(0.001)
"""


class ClockSampler:
    """SM clock and clock-event (throttle) reasons of one GPU, polled through NVML about every
    millisecond by a child process (so that this process's Python threads cannot starve it);
    `stop(t0, t1)` keeps the samples taken between two host timestamps. Read-only."""

    REASONS = {  # nvmlClocksEventReasons bits
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
    }

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        import subprocess

        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".txt", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, str(self.index)], stdout=f,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, t0_ns: int, t1_ns: int) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvml sampler could not start"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, bits, mx = [], 0, None
        for line in Path(self.path).read_text().splitlines():
            c = line.split()
            if len(c) == 2 and c[0] == "max":
                mx = float(c[1])
            elif len(c) == 3 and t0_ns <= int(c[0]) <= t1_ns:
                sm.append(float(c[1]))
                bits |= int(c[2])
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": mx, "samples": 0, "reasons": ["no NVML sample inside the timed region"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(n for b, n in self.REASONS.items() if bits & b)}


# ------------------------------------------------------------------------------------------ CPU arms
def _cpu_worker(rank, world, initfile, steps, warmup, threads, out_path, tokens):
    import torch
    import torch.distributed as dist

    from oracle import asynctp_oracle as orc

    _set_tokens(tokens)
    torch.set_num_threads(threads)
    dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    rows = CPU_SAMPLE_TOKENS // world
    x = orc.activations(rank, rows, HIDDEN, torch.float32)
    w1, w3 = orc.weights(7, HIDDEN, FFN_PER_RANK, torch.float32), orc.weights(8, HIDDEN, FFN_PER_RANK, torch.float32)
    w2 = orc.weights(9, FFN_PER_RANK, HIDDEN, torch.float32)
    h = orc.activations(50 + rank, CPU_SAMPLE_TOKENS, FFN_PER_RANK, torch.float32)

    def step():
        orc.all_gather_matmul_dist(x, [w1, w3], 0, return_A=False)
        orc.matmul_reduce_scatter_dist(h, w2, "sum", 0)

    for _ in range(warmup):
        step()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dist.barrier()
    dt = time.perf_counter() - t0
    if rank == 0:
        Path(out_path).write_text(json.dumps({"seconds": dt}))
    dist.destroy_process_group()


def cpu_unfused(world: int, steps: int, warmup: int) -> dict:
    """The reference's unfused decomposition (oracle port of autoparallel/asynctp_ops.py:672-700,
    :1090-1100) on `world` gloo ranks sharing the host cores, on CPU_SAMPLE_TOKENS of the tokens."""
    import torch.multiprocessing as mp

    cores = os.cpu_count() or 1
    threads = max(1, cores // world)
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "out.json")
        mp.spawn(_cpu_worker, args=(world, os.path.join(d, "init"), steps, warmup, threads, out, TOKENS), nprocs=world, join=True)
        dt = json.loads(Path(out).read_text())["seconds"]
    frac = CPU_SAMPLE_TOKENS / TOKENS
    ms = dt / steps * 1e3
    tflops = world * FLOPS_STEP * frac / (ms * 1e-3) / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": threads * world, "kind": "port", "ms_per_step": ms,
            "sample": f"{CPU_SAMPLE_TOKENS} of {TOKENS} tokens per step, fp32, {world} gloo rank(s) x {threads} threads, "
                      f"{steps} steps after {warmup} warm-up"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = args.gpus
    steps, warmup = max(1, args.steps), max(1, args.warmup)   # a step is ~0.1-0.5 s of host time on the 4096-token sample
    base = cpu_unfused(n, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOP/s", "n_gpus": n,
        "steps": steps, "warmup": warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config(n, "cpu"),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _config(n: int, where: str) -> dict:
    return {
        "workload": "llama3_8b_mlp_tp8_slices (BASELINE config 2)", "tokens": TOKENS, "hidden": HIDDEN,
        "ffn_per_rank": FFN_PER_RANK, "tp": n, "rows_per_rank": TOKENS // n,
        "ops": "fused_all_gather_matmul(x,[w1,w3]) + fused_matmul_reduce_scatter(h,w2)",
        "l2": "working set per step (x 268MB/tp, weights 44MB, h1/h3 235MB, h 117MB) exceeds the 126MB L2" if where == "gpu" else "n/a",
    }


# ------------------------------------------------------------------------------------------ GPU arm
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        with tempfile.TemporaryDirectory() as d:
            dist.init_process_group("gloo", init_method=f"file://{os.path.join(d, 'init')}", rank=0, world_size=1)

    from autoparallel_b200 import _native as nat
    from autoparallel_b200 import symm
    from autoparallel_b200.build import build_native
    import autoparallel_b200.asynctp_ops  # noqa: F401
    from oracle import asynctp_oracle as orc  # input generators only; nothing computes through it here

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # polls from now on; only the samples inside the timed region are kept
    build_native()
    L = nat.lib()
    ns = torch.ops._ap_symm_mem
    g = dist.group.WORLD.group_name
    rows = TOKENS // world
    K, W = args.steps, args.warmup

    x_host = orc.activations(rank, rows, HIDDEN).pin_memory()
    x = x_host.to(dev)
    w1, w3 = orc.weights(7, HIDDEN, FFN_PER_RANK).to(dev), orc.weights(8, HIDDEN, FFN_PER_RANK).to(dev)
    w2 = orc.weights(9, FFN_PER_RANK, HIDDEN).to(dev)
    _, (h1, h3) = ns.fused_all_gather_matmul(x, [w1, w3], 0, g, return_A=False)
    h = torch.nn.functional.silu(h1.float()).mul_(h3.float()).to(torch.bfloat16)
    del h1, h3

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def step():
        ns.fused_all_gather_matmul(x, [w1, w3], 0, g, return_A=False)
        ns.fused_matmul_reduce_scatter(h, w2, "sum", 0, g)

    for _ in range(max(W, 3)):
        step()
    sync_all()

    # ---- timed region: K steps, device-resident inputs; per-op events ride along on the same stream
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    launches0 = L.apk_launch_count()
    sync_all()
    t0_ns = time.time_ns()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(K):
        ev[i][0].record()
        ns.fused_all_gather_matmul(x, [w1, w3], 0, g, return_A=False)
        ev[i][1].record()
        ns.fused_matmul_reduce_scatter(h, w2, "sum", 0, g)
        ev[i][2].record()
    t_end.record()
    sync_all()
    t1_ns = time.time_ns()
    launches = L.apk_launch_count() - launches0
    clocks = sampler.stop(t0_ns, t1_ns) if rank == 0 else None
    ms_step = max_over_ranks(t_begin.elapsed_time(t_end) / K)
    ms_ag = max_over_ranks(statistics.mean(e[0].elapsed_time(e[1]) for e in ev))
    ms_rs = max_over_ranks(statistics.mean(e[1].elapsed_time(e[2]) for e in ev))
    symm.sync_check()

    # ---- end to end: every step copies its input from pinned host memory, runs both ops with the real
    #      silu*mul between them and copies the result back to pinned host memory. The copies run on
    #      their own streams, double-buffered, so the copy of step i+1 overlaps the compute of step i
    #      (what a caller feeding the op from host memory would do); the timed region ends when the last
    #      result has landed on the host.
    out_host = torch.empty(rows, HIDDEN, dtype=torch.bfloat16).pin_memory()
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty_like(x), torch.empty_like(x)]
    ev_in = [torch.cuda.Event(), torch.cuda.Event()]
    ev_free = [torch.cuda.Event(), torch.cuda.Event()]
    for e in ev_free:
        e.record(main)

    def e2e_step(i: int):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[b])            # the compute that last read this buffer is done
            x_dev[b].copy_(x_host, non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        _, (a, bb) = ns.fused_all_gather_matmul(x_dev[b], [w1, w3], 0, g, return_A=False)
        ev_free[b].record(main)
        hh = torch.nn.functional.silu(a).mul_(bb)
        o = ns.fused_matmul_reduce_scatter(hh, w2, "sum", 0, g)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out_host.copy_(o, non_blocking=True)
        o.record_stream(s_out)

    for i in range(4):
        e2e_step(i)
    main.wait_stream(s_out)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        e2e_step(i)
    main.wait_stream(s_out)
    e1.record()
    sync_all()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / K)
    symm.sync_check()

    if rank == 0:
        peak_tf, peak_kind = _peaks()
        tf_gpu = FLOPS_STEP / (ms_step * 1e-3) / 1e12
        ag_tf = FLOPS_AG / (ms_ag * 1e-3) / 1e12
        rs_tf = FLOPS_RS / (ms_rs * 1e-3) / 1e12
        nv_bytes = (world - 1) / world * TOKENS * HIDDEN * 2  # both ops move this much per GPU
        roof_ag = max(FLOPS_AG / NOMINAL_BF16, nv_bytes / NVLINK_BPS)
        roof_rs = max(FLOPS_RS / NOMINAL_BF16, nv_bytes / NVLINK_BPS)
        line = {
            "metric": METRIC, "value": tf_gpu * world, "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": max(W, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": _config(world, "gpu"),
            "per_gpu_tflops": tf_gpu,
            "ops": {
                "ag_gemm": {"ms": ms_ag, "tflops_per_gpu": ag_tf, "frac_of_north_star_roofline": roof_ag * 1e3 / ms_ag,
                            "bound": "tensor" if FLOPS_AG / NOMINAL_BF16 >= nv_bytes / NVLINK_BPS else "nvlink"},
                "gemm_rs": {"ms": ms_rs, "tflops_per_gpu": rs_tf, "frac_of_north_star_roofline": roof_rs * 1e3 / ms_rs,
                            "bound": "tensor" if FLOPS_RS / NOMINAL_BF16 >= nv_bytes / NVLINK_BPS else "nvlink"},
                "nvlink_bytes_per_gpu_per_op": nv_bytes,
            },
            "roofline": {"bound": "tensor", "kernel": _kernel_name(L), "achieved": ag_tf,
                         "peak": peak_tf, "unit": "TFLOP/s", "frac": ag_tf / peak_tf, "peak_kind": f"of {peak_kind} (sustained cuBLAS bf16)",
                         "frac_of_nominal_2250": ag_tf / 2250.0, "traffic": _traffic_ag_bytes()},
            "e2e": {"value": world * FLOPS_STEP / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": int(launches) * world,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = {k: v for k, v in cpu_unfused(1, 3, 1).items() if k != "ms_per_step"}
        print(json.dumps(line), flush=True)
    symm.shutdown()
    if world > 1:
        dist.barrier()
    dist.destroy_process_group()


# DRAM bytes (read + write) of one all-gather-mode launch at this workload, from the ncu capture
# summarised in profiles/ (8192-token capture scaled to 32768 tokens: A and outputs scale, B does not).
def _kernel_name(L) -> str:
    pair = L.apk_pair_launch_count() > 0
    return ("gemm_fused_kernel<256,6,false,true> (CTA pairs, all-gather mode)" if pair
            else "gemm_fused_kernel<256,4,false,false> (all-gather mode)")


def _traffic_ag_bytes() -> float:
    per_8192 = (99.09e6 - 29.36e6) + 41.10e6     # A read + outputs written, measured at 8192 tokens
    return 29.36e6 + per_8192 * TOKENS / 8192.0   # + B (w1, w3), read once whatever the tokens


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (used for ncu captures)")
    ap.add_argument("--tokens", type=int, default=TOKENS, help="total tokens (default: the BASELINE workload)")
    args = ap.parse_args()
    _set_tokens(args.tokens)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
