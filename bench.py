"""Benchmark of the async-TP hot path on B200: fused all-gather->matmul + matmul->reduce-scatter.

    python bench.py --gpus N --steps K --warmup W                 # this repository's kernels, headline config
    python bench.py --config attn_bf16|mlp70b_fp8|sweep|small_m   # the other BASELINE configurations
    python bench.py --impl reference --gpus N ...                 # the reference's unfused CPU path

Headline workload (BASELINE config 2, Llama-3-8B MLP at TP 8, bf16): 32768 tokens x hidden 4096 sharded
along the sequence over the N ranks; every rank holds the TP-8 weight slices w1, w3 [4096,1792] and
w2 [1792,4096] whatever N is, so the work per GPU is fixed (weak scaling). One step =
fused_all_gather_matmul(x_shard, [w1, w3]) followed by fused_matmul_reduce_scatter(h, w2) with
h [32768,1792]. Synthetic data: activations ~N(0,1) seeded by rank, weights ~N(0,0.02) (fp8: e4m3 with
row-wise / column-wise fp32 scales = amax/448). Prints ONE JSON line on rank 0.

Beside the contract keys the line carries, all measured in the same run and outside the timed region of
`value`: `parity` (both ops against an fp64 product of the same operands, the peers' inputs regenerated from
their seeds; the run fails when out of tolerance), per-op times with the same kernel on a group of one
(`local_ms`, so `exposed_comm_ms` = fused - local), the unfused NCCL + cuBLAS decomposition
(`baselines`), a loop of at least two seconds (`sustained`), and the kernel variants that ran.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL = {"bf16": 2.25e15, "fp8": 4.5e15}   # dense peaks named by the task
NVLINK_BPS = 900e9                             # per direction per GPU, nominal
METRIC = "AG+GEMM / GEMM+RS TFLOP/s (whole job; per-GPU and % of roofline beside it)"
CPU_SAMPLE_TOKENS = 4096                       # the CPU arms run this many of the tokens per step
TOL = {"bf16": 1e-2, "fp8": 3e-2}              # relative Frobenius error against fp64, as the task states them

# name -> per-GPU shapes: all-gather matmul [tokens, K] x [K, N_i]; reduce-scatter matmul [tokens, rs_K] x [rs_K, rs_N]
CONFIGS = {
    "mlp_bf16": dict(label="llama3_8b_mlp_tp8_slices (BASELINE config 2)", tokens=32768, K=4096, Ns=[1792, 1792],
                     rs_K=1792, rs_N=4096, dtype="bf16"),
    "attn_bf16": dict(label="llama3_8b_attention_projections_tp8_slices (BASELINE config 3)", tokens=32768, K=4096,
                      Ns=[512, 128, 128], rs_K=512, rs_N=4096, dtype="bf16"),
    "mlp70b_fp8": dict(label="llama3_70b_mlp_tp8_slices_fp8_rowwise (BASELINE config 4)", tokens=16384, K=8192,
                       Ns=[3584, 3584], rs_K=3584, rs_N=8192, dtype="fp8"),
}


def _flops(cfg: dict) -> tuple[float, float]:
    return 2.0 * cfg["tokens"] * cfg["K"] * sum(cfg["Ns"]), 2.0 * cfg["tokens"] * cfg["rs_K"] * cfg["rs_N"]


def _peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"burst": d.get("bf16_tflops"), "sustained": d.get("bf16_tflops_sustained"), "kind": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "kind": "fallback"}


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
    `window(t0, t1)` summarises the samples taken between two host timestamps. Read-only."""

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

    def window(self, t0_ns: int, t1_ns: int) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvml sampler could not start"]}
        sm, bits, mx = [], 0, None
        for line in Path(self.path).read_text().splitlines():
            c = line.split()
            if len(c) == 2 and c[0] == "max":
                mx = float(c[1])
            elif len(c) == 3 and t0_ns <= int(c[0]) <= t1_ns:
                sm.append(float(c[1]))
                bits |= int(c[2])
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": mx, "samples": 0, "reasons": ["no NVML sample inside the timed region"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(n for b, n in self.REASONS.items() if bits & b)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            os.unlink(self.path)
        except OSError:
            pass


# ------------------------------------------------------------------------------------------ CPU arms
def _cpu_worker(rank, world, initfile, steps, warmup, threads, out_path, cfg):
    import torch
    import torch.distributed as dist

    from oracle import asynctp_oracle as orc

    torch.set_num_threads(threads)
    dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=world)
    rows = CPU_SAMPLE_TOKENS // world
    x = orc.activations(rank, rows, cfg["K"], torch.float32)
    ws = [orc.weights(7 + i, cfg["K"], n, torch.float32) for i, n in enumerate(cfg["Ns"])]
    w2 = orc.weights(9 + len(ws), cfg["rs_K"], cfg["rs_N"], torch.float32)
    h = orc.activations(50 + rank, CPU_SAMPLE_TOKENS, cfg["rs_K"], torch.float32)

    def step():
        orc.all_gather_matmul_dist(x, ws, 0, return_A=False)
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


def cpu_unfused(cfg: dict, world: int, steps: int, warmup: int) -> dict:
    """The reference's unfused decomposition (oracle port of autoparallel/asynctp_ops.py:672-700,
    :1090-1100) on `world` gloo ranks sharing the host cores, on CPU_SAMPLE_TOKENS of the tokens, fp32."""
    import torch.multiprocessing as mp

    cores = os.cpu_count() or 1
    threads = max(1, cores // world)
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "out.json")
        mp.spawn(_cpu_worker, args=(world, os.path.join(d, "init"), steps, warmup, threads, out, cfg), nprocs=world, join=True)
        dt = json.loads(Path(out).read_text())["seconds"]
    frac = CPU_SAMPLE_TOKENS / cfg["tokens"]
    ms = dt / steps * 1e3
    tflops = world * sum(_flops(cfg)) * frac / (ms * 1e-3) / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": threads * world, "kind": "port", "ms_per_step": ms,
            "sample": f"{CPU_SAMPLE_TOKENS} of {cfg['tokens']} tokens per step, fp32, {world} gloo rank(s) x {threads} threads, "
                      f"{steps} steps after {warmup} warm-up"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = _config_for(args)
    n = args.gpus
    steps, warmup = max(1, args.steps), max(1, args.warmup)   # a step is ~0.1-0.5 s of host time on the 4096-token sample
    base = cpu_unfused(cfg, n, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOP/s", "n_gpus": n,
        "steps": steps, "warmup": warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config_json(cfg, n, "cpu"),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _config_for(args) -> dict:
    name = args.config if args.config in CONFIGS else "mlp_bf16"
    cfg = dict(CONFIGS[name])
    cfg["name"] = name
    if args.tokens:
        cfg["tokens"] = args.tokens
    return cfg


def _config_json(cfg: dict, n: int, where: str) -> dict:
    es = 1 if cfg["dtype"] == "fp8" else 2
    mb = lambda b: f"{b / 1e6:.0f}MB"   # noqa: E731
    out = {
        "workload": cfg["label"], "tokens": cfg["tokens"], "hidden": cfg["K"], "tp": n, "rows_per_rank": cfg["tokens"] // n,
        "ag_weights": cfg["Ns"], "rs_shape": [cfg["rs_K"], cfg["rs_N"]],
        "ops": "fused_all_gather_matmul(x,Bs) + fused_matmul_reduce_scatter(h,w2)" if cfg["dtype"] == "bf16"
               else "fused_all_gather_scaled_matmul(x8,Bs8,row scales) + fused_scaled_matmul_reduce_scatter(h8,w2_8)",
        "l2": (f"working set per step (x {mb(cfg['tokens'] * cfg['K'] * es)}/tp, AG outputs {mb(cfg['tokens'] * sum(cfg['Ns']) * 2)}, "
               f"h {mb(cfg['tokens'] * cfg['rs_K'] * es)}) exceeds the 126MB L2") if where == "gpu" else "n/a",
    }
    if cfg["name"] == "mlp_bf16":
        out["ffn_per_rank"] = cfg["Ns"][0]
    return out


# ------------------------------------------------------------------------------------------ GPU arm
def _randn(shape, seed: int, dev, std: float = 1.0):
    """Seeded N(0, std) on the device (Philox: the same values on every GPU of the box for one seed)."""
    import torch

    g = torch.Generator(device=dev).manual_seed(seed)
    t = torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
    return t if std == 1.0 else t.mul_(std)


def _quant_rows(x):
    """e4m3 with one fp32 scale per row: scale = amax/448 (BASELINE config 4)."""
    import torch

    s = x.abs().amax(dim=1, keepdim=True).clamp_min(1e-12) / 448.0
    return (x / s).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn), s


class Workload:
    """Device-resident inputs of one configuration on this rank, and the calls that run it."""

    def __init__(self, cfg: dict, rank: int, world: int, dev, group_name: str):
        import torch

        self.cfg, self.rank, self.world, self.dev, self.g = cfg, rank, world, dev, group_name
        self.fp8 = cfg["dtype"] == "fp8"
        self.rows = cfg["tokens"] // world
        self.ns = torch.ops._ap_symm_mem
        bf = torch.bfloat16
        self.x_f32 = None
        x = self.shard_x(rank)
        h = self.full_h(rank)
        Bs = [_randn((cfg["K"], n), 7 + i, dev, 0.02) for i, n in enumerate(cfg["Ns"])]
        w2 = _randn((cfg["rs_K"], cfg["rs_N"]), 9 + len(Bs), dev, 0.02)
        if self.fp8:
            self.x, self.x_scale = _quant_rows(x)
            self.h, self.h_scale = _quant_rows(h)
            qb = [_quant_rows(b.t().contiguous()) for b in Bs]           # per column of B = per row of B^T
            self.Bs = [q.t() for q, _ in qb]                              # [K, N] views with K contiguous
            self.B_scales = [s.t().contiguous() for _, s in qb]           # [1, N]
            q2, s2 = _quant_rows(w2.t().contiguous())
            self.w2, self.w2_scale = q2.t(), s2.t().contiguous()
        else:
            self.x, self.h = x.to(bf), h.to(bf)
            self.Bs = [b.to(bf) for b in Bs]
            self.w2 = w2.to(bf)
        del x, h, Bs, w2

    # -- seeded inputs of any rank (used for this rank's tensors and, in the parity check, for the peers')
    def shard_x(self, r: int):
        return _randn((self.rows, self.cfg["K"]), 1000 + r, self.dev)

    def full_h(self, r: int):
        return _randn((self.cfg["tokens"], self.cfg["rs_K"]), 50 + r, self.dev)

    # -- the two ops on group `g` (default: the tensor-parallel group)
    def ag(self, x=None, x_scale=None, g=None):
        import torch

        x = self.x if x is None else x
        g = g or self.g
        if self.fp8:
            n = len(self.Bs)
            return self.ns.fused_all_gather_scaled_matmul(x, self.Bs, self.x_scale if x_scale is None else x_scale, self.B_scales, 0, g,
                                                          [None] * n, [None] * n, [torch.bfloat16] * n, [False] * n)[1]
        return self.ns.fused_all_gather_matmul(x, self.Bs, 0, g, return_A=False)[1]

    def rs(self, h=None, h_scale=None, g=None):
        import torch

        h = self.h if h is None else h
        g = g or self.g
        if self.fp8:
            return self.ns.fused_scaled_matmul_reduce_scatter(h, self.w2, self.h_scale if h_scale is None else h_scale, self.w2_scale,
                                                              "sum", 0, 0, g, [h.shape[0], self.cfg["rs_N"]], None, None, torch.bfloat16, False)
        return self.ns.fused_matmul_reduce_scatter(h, self.w2, "sum", 0, g)

    # -- fp64 views of operands (dequantised for fp8)
    def deq(self, q, scale=None):
        import torch

        d = q.to(torch.float64)
        return d if scale is None else d * scale.to(torch.float64)


def _freivalds(out, rhs_fn, n_out: int, dev, seed: int) -> float:
    """||out V - ref V||_F / ||ref V||_F for four random vectors V, ref V computed in fp64 by rhs_fn(V)."""
    import torch

    V = _randn((n_out, 4), seed, dev).to(torch.float64)
    lhs = out.to(torch.float64) @ V
    rhs = rhs_fn(V)
    return ((lhs - rhs).norm() / rhs.norm().clamp_min(1e-300)).item()


def parity_check(w: Workload) -> dict:
    """Both ops against fp64 products of the same (quantised) operands, the peers' inputs regenerated from
    their seeds. Freivalds' check on the full outputs: out @ V against A @ (B @ V)."""
    import torch

    cfg = w.cfg
    outs = w.ag()
    red = w.rs()
    torch.cuda.synchronize()
    # gathered A in fp64, rank by rank
    parts = []
    for r in range(w.world):
        xr = w.shard_x(r)
        if w.fp8:
            q, s = _quant_rows(xr)
            parts.append(w.deq(q, s))
        else:
            parts.append(xr.to(torch.bfloat16).to(torch.float64))
        del xr
    A = torch.cat(parts)
    del parts
    ag_err = 0.0
    for i, (o, B) in enumerate(zip(outs, w.Bs)):
        Bd = w.deq(B, w.B_scales[i]) if w.fp8 else B.to(torch.float64)
        ag_err = max(ag_err, _freivalds(o, lambda V: A @ (Bd @ V), B.shape[1], w.dev, 4000 + i))
    del A
    W2 = w.deq(w.w2, w.w2_scale) if w.fp8 else w.w2.to(torch.float64)
    lo = w.rank * (cfg["tokens"] // w.world)
    hi = lo + cfg["tokens"] // w.world

    def rs_ref(V):
        acc = None
        WV = W2 @ V
        for r in range(w.world):
            hr = w.full_h(r)
            if w.fp8:
                q, s = _quant_rows(hr)
                part = w.deq(q[lo:hi], s[lo:hi]) @ WV
            else:
                part = hr[lo:hi].to(torch.bfloat16).to(torch.float64) @ WV
            acc = part if acc is None else acc + part
            del hr
        return acc

    rs_err = _freivalds(red, rs_ref, cfg["rs_N"], w.dev, 4100)
    tol = TOL[cfg["dtype"]]
    return {"ag_rel_err": ag_err, "rs_rel_err": rs_err, "tol": tol, "ok": bool(ag_err <= tol and rs_err <= tol and math.isfinite(ag_err + rs_err)),
            "how": "Freivalds (4 vectors) on the full outputs against fp64 products of the same operands; peers' inputs regenerated from their seeds"}


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
    tmpdir = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        tmpdir = tempfile.TemporaryDirectory()
        dist.init_process_group("gloo", init_method=f"file://{os.path.join(tmpdir.name, 'init')}", rank=0, world_size=1)

    from autoparallel_b200 import _native as nat
    from autoparallel_b200 import symm
    from autoparallel_b200.build import build_native
    import autoparallel_b200.asynctp_ops  # noqa: F401

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # polls from now on; only the samples inside the timed regions are kept
    build_native()
    L = nat.lib()
    g = dist.group.WORLD.group_name
    solo = g
    if world > 1:                # a group of one per rank: the same kernels without peers ("local")
        for r in range(world):
            gr = dist.new_group([r])
            if r == rank:
                solo = gr.group_name

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

    def time_call(fn, iters: int, warm: int = 3) -> float:
        """ms per call, CUDA events on the current stream, max over ranks."""
        for _ in range(warm):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        sync_all()
        return max_over_ranks(e0.elapsed_time(e1) / iters)

    if args.config in ("sweep", "small_m"):
        _run_sweep(args, rank, world, dev, g, solo, time_call, L, symm, sampler)
    else:
        _run_config(args, rank, world, dev, g, solo, sync_all, max_over_ranks, time_call, L, symm, sampler)
    sampler.stop()
    symm.shutdown()
    if world > 1:
        dist.barrier()
    dist.destroy_process_group()
    if tmpdir is not None:
        tmpdir.cleanup()


def _unfused(w: Workload, dist, torch):
    """The reference's unfused decomposition on the GPU (autoparallel/asynctp_ops.py:672-700, :1090-1100 and the
    scaled forms): NCCL all_gather_into_tensor / reduce_scatter_tensor + torch.mm / torch._scaled_mm."""
    cfg = w.cfg
    M = cfg["tokens"]
    gathered = torch.empty((M, cfg["K"]), dtype=w.x.dtype, device=w.dev)
    gathered_scale = torch.empty((M, 1), dtype=torch.float32, device=w.dev) if w.fp8 else None
    red = torch.empty((M // w.world, cfg["rs_N"]), dtype=torch.bfloat16, device=w.dev)

    def ag():
        if w.world > 1:
            dist.all_gather_into_tensor(gathered.view(torch.uint8) if w.fp8 else gathered, w.x.view(torch.uint8) if w.fp8 else w.x)
            if w.fp8:
                dist.all_gather_into_tensor(gathered_scale, w.x_scale)
            A, As = gathered, gathered_scale
        else:
            A, As = w.x, (w.x_scale if w.fp8 else None)
        if w.fp8:
            return [torch._scaled_mm(A, B, As, bs, out_dtype=torch.bfloat16) for B, bs in zip(w.Bs, w.B_scales)]
        return [torch.mm(A, B) for B in w.Bs]

    def rs():
        full = torch._scaled_mm(w.h, w.w2, w.h_scale, w.w2_scale, out_dtype=torch.bfloat16) if w.fp8 else torch.mm(w.h, w.w2)
        if w.world > 1:
            dist.reduce_scatter_tensor(red, full)
            return red
        return full

    return ag, rs


def _run_config(args, rank, world, dev, g, solo, sync_all, max_over_ranks, time_call, L, symm, sampler) -> None:
    import torch
    import torch.distributed as dist

    cfg = _config_for(args)
    K, W = args.steps, max(args.warmup, 3)
    fl_ag, fl_rs = _flops(cfg)
    w = Workload(cfg, rank, world, dev, g)

    for _ in range(W):
        w.ag()
        w.rs()
    sync_all()

    # ---- parity, outside every timed region; a run that computes the wrong thing has no number
    parity = parity_check(w)
    ok = torch.tensor([1.0 if parity["ok"] else 0.0, parity["ag_rel_err"], parity["rs_rel_err"]], device=dev, dtype=torch.float64)
    if world > 1:
        worst = ok.clone()
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        parity["ag_rel_err"], parity["rs_rel_err"] = worst[1].item(), worst[2].item()
        parity["ok"] = bool(ok[0].item() > 0.5)
    symm.sync_check()
    if not parity["ok"]:
        if rank == 0:
            print(json.dumps({"error": "parity check failed", "parity": parity, "config": _config_json(cfg, world, "gpu")}), flush=True)
        raise SystemExit(3)

    # ---- timed region: K steps, device-resident inputs; per-op events ride along on the same stream
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    launches0, pairs0 = L.apk_launch_count(), L.apk_pair_launch_count()
    sync_all()
    t0_ns = time.time_ns()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(K):
        ev[i][0].record()
        w.ag()
        ev[i][1].record()
        w.rs()
        ev[i][2].record()
    t_end.record()
    sync_all()
    t1_ns = time.time_ns()
    launches, pairs = L.apk_launch_count() - launches0, L.apk_pair_launch_count() - pairs0
    ms_step = max_over_ranks(t_begin.elapsed_time(t_end) / K)
    ms_ag = max_over_ranks(statistics.mean(e[0].elapsed_time(e[1]) for e in ev))
    ms_rs = max_over_ranks(statistics.mean(e[1].elapsed_time(e[2]) for e in ev))
    symm.sync_check()

    # ---- the same kernels on a group of one (all rows local): fused - local = exposed communication
    ms_ag_local = ms_rs_local = None
    if world > 1 and not args.quick:
        xf = torch.cat([w.x] * world)
        xs = torch.cat([w.x_scale] * world) if w.fp8 else None
        ms_ag_local = time_call(lambda: w.ag(xf, xs, solo), 10)
        ms_rs_local = time_call(lambda: w.rs(g=solo), 10)
        del xf, xs

    # ---- GPU baseline: the unfused NCCL + cuBLAS decomposition
    baselines = None
    if not args.quick:
        uag, urs = _unfused(w, dist, torch)
        baselines = {"unfused_nccl_cublas": {"ag_ms": time_call(uag, 10), "rs_ms": time_call(urs, 10),
                                             "what": "all_gather_into_tensor + torch.mm / _scaled_mm; mm + reduce_scatter_tensor (NCCL)"},
                     "reference_cuda_path": {"unavailable": "the reference package cannot be installed offline (its build backend, "
                                             "hatchling, is absent), so its sources are not where this benchmark runs"}}

    # ---- a loop of at least two seconds: the clock settles under the power cap
    sustained = None
    if not args.quick:
        n_sus = max(K, int(math.ceil(2000.0 / ms_step)))
        sync_all()
        s0_ns = time.time_ns()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_sus):
            w.ag()
            w.rs()
        e1.record()
        sync_all()
        s1_ns = time.time_ns()
        ms_sus = max_over_ranks(e0.elapsed_time(e1) / n_sus)
        symm.sync_check()
        sustained = {"steps": n_sus, "ms_per_step": ms_sus, "tflops_per_gpu": (fl_ag + fl_rs) / (ms_sus * 1e-3) / 1e12,
                     "seconds": ms_sus * n_sus / 1e3}
        if rank == 0:
            sustained["clocks"] = sampler.window(s0_ns, s1_ns)

    # ---- end to end: every step copies its input from pinned host memory, runs both ops with the real
    #      silu*mul (and, for fp8, the row-wise re-quantisation) between them and copies the result back to
    #      pinned host memory. The copies run on their own streams, double-buffered, so the copy of step i+1
    #      overlaps the compute of step i; the timed region ends when the last result has landed on the host.
    x_host = w.x.cpu().pin_memory()
    xs_host = w.x_scale.cpu().pin_memory() if w.fp8 else None
    out_host = torch.empty(w.rows, cfg["rs_N"], dtype=torch.bfloat16).pin_memory()
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty_like(w.x), torch.empty_like(w.x)]
    xs_dev = [torch.empty_like(w.x_scale), torch.empty_like(w.x_scale)] if w.fp8 else None
    ev_in = [torch.cuda.Event(), torch.cuda.Event()]
    ev_free = [torch.cuda.Event(), torch.cuda.Event()]
    for e in ev_free:
        e.record(main)
    pair_out = len(cfg["Ns"]) == 2 and cfg["Ns"][0] == cfg["Ns"][1] == cfg["rs_K"]

    def e2e_step(i: int):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[b])            # the compute that last read this buffer is done
            x_dev[b].copy_(x_host, non_blocking=True)
            if w.fp8:
                xs_dev[b].copy_(xs_host, non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        outs = w.ag(x_dev[b], xs_dev[b] if w.fp8 else None)
        ev_free[b].record(main)
        if pair_out:
            hh = torch.nn.functional.silu(outs[0]).mul_(outs[1])
        else:
            hh = outs[0][:, : cfg["rs_K"]].contiguous()   # attention: the q projection stands in for the attention output
        if w.fp8:
            hq, hs = _quant_rows(hh.float())
            o = w.rs(hq, hs)
        else:
            o = w.rs(hh)
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
    h2d = x_host.numel() * x_host.element_size() + (xs_host.numel() * 4 if w.fp8 else 0)

    if rank == 0:
        peaks = _peaks()
        dt = cfg["dtype"]
        peak_scale = 2.0 if dt == "fp8" else 1.0
        nominal = NOMINAL[dt]
        tf_gpu = (fl_ag + fl_rs) / (ms_step * 1e-3) / 1e12
        ag_tf = fl_ag / (ms_ag * 1e-3) / 1e12
        rs_tf = fl_rs / (ms_rs * 1e-3) / 1e12
        es = 1 if dt == "fp8" else 2
        nv_ag = (world - 1) / world * cfg["tokens"] * (cfg["K"] * es + (4 if dt == "fp8" else 0))
        nv_rs = (world - 1) / world * cfg["tokens"] * cfg["rs_N"] * 2
        roof_ag = max(fl_ag / nominal, nv_ag / NVLINK_BPS)
        roof_rs = max(fl_rs / nominal, nv_rs / NVLINK_BPS)

        def op_line(ms, tf, fl, nv, roof, local):
            d = {"ms": ms, "tflops_per_gpu": tf, "frac_of_north_star_roofline": roof * 1e3 / ms,
                 "bound": "tensor" if fl / nominal >= nv / NVLINK_BPS else "nvlink",
                 "nvlink_bytes_per_gpu": nv, "nvlink_gbs_per_gpu": nv / (ms * 1e-3) / 1e9}
            if local is not None:
                d["local_ms"] = local
                d["exposed_comm_ms"] = ms - local
            return d

        burst = peaks["burst"] * peak_scale
        line = {
            "metric": METRIC, "value": tf_gpu * world, "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dt == "bf16" else "e4m3 (fp32 accumulate, bf16 out)",
            "data": "synthetic", "config": _config_json(cfg, world, "gpu"),
            "per_gpu_tflops": tf_gpu,
            "parity": parity,
            "ops": {"ag_gemm": op_line(ms_ag, ag_tf, fl_ag, nv_ag, roof_ag, ms_ag_local),
                    "gemm_rs": op_line(ms_rs, rs_tf, fl_rs, nv_rs, roof_rs, ms_rs_local)},
            "kernels": {"launches_timed": int(launches), "as_cta_pairs": int(pairs), "pairs_refused_by_device": int(L.apk_pair_refusal_count()),
                        "variant": _kernel_name(cfg, pairs > 0)},
            "roofline": {"bound": "tensor", "kernel": _kernel_name(cfg, pairs > 0) + ", all-gather mode", "achieved": ag_tf,
                         "peak": burst, "unit": "TFLOP/s", "frac": ag_tf / burst,
                         "peak_kind": f"of {peaks['kind']} cuBLAS bf16 burst peak" + (" x 2 for e4m3 (no fp8 figure in MEASURED_PEAKS.json)" if dt == "fp8" else "")
                                      + ": the timed region is tens of milliseconds",
                         "frac_of_nominal": ag_tf * 1e12 / nominal, "traffic": _traffic_ag_bytes(cfg),
                         "traffic_source": "ncu dram__bytes of the 8192-token capture of this kernel variant (profiles/), A and outputs scaled to the tokens"},
            "e2e": {"value": world * (fl_ag + fl_rs) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": out_host.numel() * 2,
                    "note": "bound by the host link, not by the kernels: the copies are overlapped with compute and take longer than it"},
            "gpu_launches": int(launches) * world,
            "clocks": sampler.window(t0_ns, t1_ns),
        }
        if sustained is not None:
            sustained["frac_of_sustained_peak"] = sustained["tflops_per_gpu"] / (peaks["sustained"] * peak_scale)
            sustained["peak"] = peaks["sustained"] * peak_scale
            line["sustained"] = sustained
        if baselines is not None:
            line["baselines"] = baselines
        if world == 1 and not args.no_cpu_baseline and not args.quick:
            line["cpu_baseline"] = {k: v for k, v in cpu_unfused(cfg, 1, 3, 1).items() if k != "ms_per_step"}
        print(json.dumps(line), flush=True)


def _run_sweep(args, rank, world, dev, g, solo, time_call, L, symm, sampler) -> None:
    """BASELINE config 5 (`sweep`: total M in 2048..65536, K = N in {4096, 8192}) or the small-M regime the reference
    serves with its native / multimem shortcuts (`small_m`: M in 256..4096; autoparallel/asynctp_ops.py:770-772,
    :852-854). Per point: fused, the same kernel on a group of one, and the unfused NCCL + cuBLAS decomposition."""
    import torch
    import torch.distributed as dist

    Ms = [2048 << i for i in range(6)] if args.config == "sweep" else [256, 512, 1024, 2048, 4096]
    points = []
    iters = max(5, args.steps)
    for KN in (4096, 8192):
        for M in Ms:
            if M % (world * 8) != 0:
                continue
            cfg = dict(name="sweep", label=f"sweep M={M} K=N={KN}", tokens=M, K=KN, Ns=[KN], rs_K=KN, rs_N=KN, dtype="bf16")
            w = Workload(cfg, rank, world, dev, g)
            par = parity_check(w) if M <= 8192 else None
            fl = 2.0 * M * KN * KN
            ag = time_call(w.ag, iters)
            rs = time_call(w.rs, iters)
            xf = torch.cat([w.x] * world)
            ag_l = time_call(lambda: w.ag(xf, None, solo), iters)
            rs_l = time_call(lambda: w.rs(g=solo), iters)
            uag, urs = _unfused(w, dist, torch)
            ag_u, rs_u = time_call(uag, iters), time_call(urs, iters)
            nv = (world - 1) / world * M * KN * 2
            roof = max(fl / NOMINAL["bf16"], nv / NVLINK_BPS) * 1e3
            pt = {"M": M, "K": KN, "N": KN,
                  "ag_gemm": {"ms": ag, "tflops_per_gpu": fl / ag / 1e9, "frac_of_north_star_roofline": roof / ag, "local_ms": ag_l,
                              "exposed_comm_ms": ag - ag_l, "unfused_ms": ag_u, "unfused_exposed_comm_ms": ag_u - ag_l},
                  "gemm_rs": {"ms": rs, "tflops_per_gpu": fl / rs / 1e9, "frac_of_north_star_roofline": roof / rs, "local_ms": rs_l,
                              "exposed_comm_ms": rs - rs_l, "unfused_ms": rs_u, "unfused_exposed_comm_ms": rs_u - rs_l}}
            if par is not None:
                pt["parity"] = {k: par[k] for k in ("ag_rel_err", "rs_rel_err", "ok")}
                if not par["ok"]:
                    raise SystemExit(3)
            points.append(pt)
            symm.sync_check()
            del w, xf
            torch.cuda.empty_cache()
    if rank == 0:
        head = next((p for p in points if p["M"] == 32768 and p["K"] == 4096), points[-1])
        tf = (head["ag_gemm"]["tflops_per_gpu"] + head["gemm_rs"]["tflops_per_gpu"]) / 2
        print(json.dumps({
            "metric": METRIC, "value": tf * world, "unit": "TFLOP/s", "n_gpus": world, "steps": iters, "warmup": 3,
            "ms_per_step": head["ag_gemm"]["ms"] + head["gemm_rs"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"shape {args.config} (BASELINE config 5 / small-M regime); value = mean of the two ops at M={head['M']}, K=N={head['K']}",
                       "tp": world, "l2": "every point is timed back to back; points with M*K*2 below 126MB stay L2-resident"},
            "sweep": points, "gpu_launches": int(L.apk_launch_count()) * world,
        }), flush=True)


def _kernel_name(cfg: dict, pair: bool) -> str:
    fp8 = "true" if cfg["dtype"] == "fp8" else "false"
    return (f"gemm_fused_kernel<256,6,{fp8},true> (CTA pairs)" if pair else f"gemm_fused_kernel<256,4 or 128,6,{fp8},false> (single CTAs)")


def _traffic_ag_bytes(cfg: dict):
    """DRAM bytes (read + write) of one all-gather-mode launch of the headline workload: measured with ncu at 8192
    tokens on the CTA-pair kernel (profiles/), A and the outputs scaled to the tokens, B read once whatever they are."""
    if cfg["name"] != "mlp_bf16":
        return None
    return _NCU_B_BYTES + (_NCU_8192_READ - _NCU_B_BYTES + _NCU_8192_WRITE) * cfg["tokens"] / 8192.0


_NCU_B_BYTES = 29.36e6        # w1 + w3
_NCU_8192_READ = 104.65e6     # dram__bytes_read.sum at 8192 tokens
_NCU_8192_WRITE = 42.38e6     # dram__bytes_write.sum at 8192 tokens


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=[*CONFIGS, "sweep", "small_m"], default="mlp_bf16",
                    help="mlp_bf16 is the headline (BASELINE config 2); the others are the remaining BASELINE configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg")
    ap.add_argument("--quick", action="store_true", help="only parity, the timed steps and the end-to-end loop (ncu captures)")
    ap.add_argument("--tokens", type=int, default=0, help="total tokens (default: the configuration's own)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
