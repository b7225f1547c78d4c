"""Generates tests/golden/asynctp_golden.pt by running the REFERENCE's own unfused fallbacks.

Run where the AutoParallel sources are available (the fixtures it writes are what travels with this repository):

    python tests/golden/make_golden.py /path/to/autoparallel_checkout

Two gloo ranks on CPU import the reference's ``autoparallel.asynctp_ops`` unmodified and call
its Meta/fallback kernels directly (the dispatcher has no CPU key for them):
``_fused_all_gather_matmul_fallback``, ``_fused_matmul_reduce_scatter_fallback`` and, with
tensor-wise scales (the only scaling CPU ``torch._scaled_mm`` accepts),
``_fused_scaled_matmul_reduce_scatter_fallback``. ``_fused_all_gather_scaled_matmul_fallback``
cannot run over gloo, which has no fp8 all-gather: ``make_golden_fp8.py`` beside this file covers it
over an in-process threaded process group.
Inputs and every rank's outputs are stored, so the oracle tests need neither the reference nor
a matching RNG.
"""
import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

WORLD = 2
OUT = Path(__file__).resolve().parent / "asynctp_golden.pt"
FP8 = torch.float8_e4m3fn


def _rand(seed, *shape, dtype=torch.float32, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def _cases():
    cases = []
    # ---- all-gather -> matmul (asynctp_ops.py:672-700)
    for dtype in (torch.float32, torch.bfloat16):
        for shape, gd in (((48, 64), 0), ((4, 6, 64), 0), ((4, 6, 64), 1), ((4, 6, 64), 2)):
            K = shape[-1] * (WORLD if gd == len(shape) - 1 else 1)
            cases.append(dict(kind="ag_mm", dtype=dtype, shape=shape, gather_dim=gd, K=K, Ns=(40, 24)))
    # ---- matmul -> reduce-scatter (asynctp_ops.py:1090-1100)
    for dtype in (torch.float32, torch.bfloat16):
        for shape, sd in (((48, 64), 0), ((4, 6, 64), 0), ((4, 6, 64), 1)):
            for op in ("sum", "avg"):
                cases.append(dict(kind="mm_rs", dtype=dtype, shape=shape, scatter_dim=sd, N=40, op=op))
    # ---- fp8, tensor-wise scales
    # (the scaled all-gather fallback cannot run here: gloo rejects fp8 payloads with
    #  "Invalid scalar type" at asynctp_ops.py:889-892, so only the reduce-scatter side is pinned)
    cases.append(dict(kind="smm_rs", shape=(64, 64), N=48, op="sum"))
    cases.append(dict(kind="smm_rs", shape=(64, 64), N=48, op="avg"))
    # ---- BASELINE config 1 at full size (digest only)
    cases.append(dict(kind="config1"))
    return cases


def _digest(t):
    f = t.flatten().double()
    idx = torch.arange(0, f.numel(), 509)
    return dict(shape=tuple(t.shape), sum=f.sum().item(), abs_sum=f.abs().sum().item(), sample=t.flatten()[idx].clone())


def _worker(rank, ref_root, initfile, outdir):
    sys.path.insert(0, ref_root)
    dist.init_process_group("gloo", init_method=f"file://{initfile}", rank=rank, world_size=WORLD)
    torch.set_num_threads(2)
    import autoparallel.asynctp_ops as ref

    g = dist.group.WORLD.group_name
    records = []
    for ci, c in enumerate(_cases()):
        rec = dict(c)
        if c["kind"] == "ag_mm":
            A = _rand(100 * ci + rank, *c["shape"], dtype=c["dtype"])
            Bs = [_rand(100 * ci + 50 + i, c["K"], n, dtype=c["dtype"], std=0.05) for i, n in enumerate(c["Ns"])]
            Aout, outs = ref._fused_all_gather_matmul_fallback(A, Bs, c["gather_dim"], g, return_A=True)
            rec.update(A_shard=A, Bs=Bs, A_out=Aout, outs=outs)
        elif c["kind"] == "mm_rs":
            A = _rand(100 * ci + rank, *c["shape"], dtype=c["dtype"])
            B = _rand(100 * ci + 50 + rank, c["shape"][-1], c["N"], dtype=c["dtype"], std=0.05)
            out = ref._fused_matmul_reduce_scatter_fallback(A, B, c["op"], c["scatter_dim"], g)
            rec.update(A=A, B=B, out=out)
        elif c["kind"] == "smm_rs":
            A = _rand(100 * ci + rank, *c["shape"]).to(FP8)
            B = _rand(100 * ci + 50 + rank, c["N"], c["shape"][-1], std=0.5).to(FP8).t()
            sa = torch.tensor(0.75 + rank)
            sb = torch.tensor(0.5)
            out = ref._fused_scaled_matmul_reduce_scatter_fallback(
                A, B, sa, sb, c["op"], 0, 0, g, [c["shape"][0], c["N"]], None, None, torch.bfloat16, False
            )
            rec.update(A=A, B_t=B.t().contiguous(), A_scale=sa, B_scale=sb, out=out)
        elif c["kind"] == "config1":
            # fp32 [512,1024] ~N(0,1) seeded by rank; B [1024,2048] and W2 [2048,1024] ~N(0,0.02), same on all ranks
            A = _rand(1000 + rank, 512, 1024)
            B = _rand(7, 1024, 2048, std=0.02)
            W2 = _rand(8, 2048, 1024, std=0.02)
            _, (C1,) = ref._fused_all_gather_matmul_fallback(A, [B], 0, g, return_A=False)
            out = ref._fused_matmul_reduce_scatter_fallback(C1, W2, "sum", 0, g)
            rec.update(C_digest=_digest(C1), out_digest=_digest(out))
        records.append(rec)
    torch.save(records, os.path.join(outdir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AUTOPARALLEL_REFERENCE", "")
    if not os.path.isdir(ref_root):
        raise SystemExit("usage: pass the AutoParallel source tree as the first argument (or in $AUTOPARALLEL_REFERENCE)")
    with tempfile.TemporaryDirectory() as d:
        initfile = os.path.join(d, "init")
        mp.spawn(_worker, args=(ref_root, initfile, d), nprocs=WORLD, join=True)
        per_rank = [torch.load(os.path.join(d, f"rank{r}.pt"), weights_only=False) for r in range(WORLD)]
    for r in per_rank:
        for rec in r:
            rec["dtype"] = str(rec.get("dtype", ""))
    torch.save(dict(world=WORLD, torch=torch.__version__, ranks=per_rank), OUT)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(per_rank[0])} cases)")


if __name__ == "__main__":
    main()
