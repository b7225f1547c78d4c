"""Generates tests/golden/asynctp_golden_fp8.pt: the REFERENCE's scaled (fp8) fallbacks on CPU.

    python tests/golden/make_golden_fp8.py /path/to/autoparallel_checkout

``make_golden.py`` runs the reference over gloo, which cannot move fp8 payloads, so the scaled
all-gather fallback (autoparallel/asynctp_ops.py:873-944) is missing there. This script runs two
ranks as THREADS of one process over torch's in-process "threaded" process group
(torch.testing._internal.distributed.multi_threaded_pg), whose collectives copy tensors of any
dtype, and calls the reference's ``_fused_all_gather_scaled_matmul_fallback`` and
``_fused_scaled_matmul_reduce_scatter_fallback`` unmodified.

Two groups of cases, marked by ``scaled_mm`` in every record:

* ``"torch-cpu"``: tensor-wise scales. Everything, ``aten::_scaled_mm`` included, is the
  reference's call into stock torch.
* ``"stand-in"``: row-wise scales (sharded and replicated) and the row-wise reduce-scatter. CPU
  ``aten::_scaled_mm`` rejects non-scalar scales, so for these cases only, and in this process
  only, a CPU kernel is registered for it that computes the documented row-wise result in fp32:
  ``((A @ B) * scale_a[:, None] * scale_b[None, :] + bias) * scale_result -> out_dtype``. What these cases
  pin is the reference's own plumbing around that call: which scale mode it detects, how it
  gathers and re-orders A and the row scales for every gather_dim, the views and movedims of the
  results, ``output_shape`` and the reduce-scatter. The row-wise arithmetic itself is checked
  against ``torch._scaled_mm`` on a GPU by the gpu tests.
"""
import os
import sys
import threading
import traceback
from pathlib import Path

import torch
import torch.distributed as dist

WORLD = 2
OUT = Path(__file__).resolve().parent / "asynctp_golden_fp8.pt"
FP8 = torch.float8_e4m3fn
BF16 = torch.bfloat16


def _rand(seed, *shape, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * std


def _colmajor(t):
    return t.t().contiguous().t()


def _cases():
    cases = []
    # ---- all-gather -> scaled matmul, tensor-wise scales (stock CPU _scaled_mm)
    for shape, gd in (((16, 32), 0), ((2, 8, 32), 0), ((2, 8, 32), 1)):
        cases.append(dict(kind="sag_mm", scaled_mm="torch-cpu", mode="tensor", shape=shape, gather_dim=gd, Ns=(48, 16),
                          out_dtypes=(BF16, torch.float32), bias=False, result_scale=False))
    # ---- row-wise scales (stand-in kernel for the row-wise arithmetic)
    for mode in ("row_sharded", "row_replicated"):
        for shape, gd in (((16, 32), 0), ((2, 8, 32), 0), ((2, 8, 32), 1)):
            cases.append(dict(kind="sag_mm", scaled_mm="stand-in", mode=mode, shape=shape, gather_dim=gd, Ns=(48, 16),
                              out_dtypes=(BF16, torch.float32), bias=(mode == "row_sharded"), result_scale=(gd == 1)))
    # ---- scaled matmul -> reduce-scatter, row-wise, 2-D and 3-D with scatter along dim 0 and 1
    for shape, sd, op in (((32, 32), 0, "sum"), ((4, 8, 32), 0, "avg"), ((4, 8, 32), 1, "sum")):
        cases.append(dict(kind="smm_rs", scaled_mm="stand-in", mode="row", shape=shape, scatter_dim=sd, N=48, op=op))
    return cases


def _scaled_mm_rowwise_cpu(a, b, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None, use_fast_accum=False):
    acc = a.float() @ b.float()
    acc = acc * scale_a.float().reshape(-1, 1) if scale_a.numel() > 1 else acc * scale_a.float()
    acc = acc * scale_b.float().reshape(1, -1) if scale_b.numel() > 1 else acc * scale_b.float()
    if bias is not None:
        acc = acc + bias.float().reshape(1, -1)
    if scale_result is not None:
        acc = acc * scale_result.float()
    return acc.to(out_dtype or a.dtype)


def _run_case(ref, ci, c, rank, g):
    rec = dict(c)
    if c["kind"] == "sag_mm":
        shape, gd = c["shape"], c["gather_dim"]
        K = shape[-1]
        A = _rand(100 * ci + rank, *shape).to(FP8)
        Bs = [_colmajor(_rand(100 * ci + 50 + i, K, n, std=0.5).to(FP8)) for i, n in enumerate(c["Ns"])]
        if c["mode"] == "tensor":
            A_scale = torch.tensor(0.75)
            B_scales = [torch.tensor(0.5 + 0.25 * i) for i in range(len(Bs))]
        else:
            B_scales = [torch.rand(1, n, generator=torch.Generator().manual_seed(100 * ci + 70 + i)) + 0.5 for i, n in enumerate(c["Ns"])]
            per_rank = [torch.rand(*shape[:-1], 1, generator=torch.Generator().manual_seed(100 * ci + 80 + r)) + 0.5 for r in range(WORLD)]
            A_scale = per_rank[rank] if c["mode"] == "row_sharded" else torch.cat(per_rank, dim=gd)
        biases = [(_rand(100 * ci + 90 + i, n).to(BF16) if c["bias"] else None) for i, n in enumerate(c["Ns"])]
        result_scales = [(torch.tensor(1.5) if c["result_scale"] else None) for _ in Bs]
        A_out, outs = ref._fused_all_gather_scaled_matmul_fallback(
            A, Bs, A_scale, B_scales, gd, g, biases, result_scales, list(c["out_dtypes"]), [False] * len(Bs)
        )
        rec.update(A_shard=A, Bs_t=[B.t().contiguous() for B in Bs], A_scale=A_scale, B_scales=B_scales,
                   biases=biases, result_scales=result_scales, A_out=A_out.contiguous(), outs=[o.contiguous() for o in outs])
    else:
        shape, sd = c["shape"], c["scatter_dim"]
        K, N = shape[-1], c["N"]
        A = _rand(100 * ci + rank, *shape).to(FP8)
        B = _colmajor(_rand(100 * ci + 50 + rank, K, N, std=0.5).to(FP8))
        A_scale = torch.rand(*shape[:-1], 1, generator=torch.Generator().manual_seed(100 * ci + 80 + rank)) + 0.5
        B_scale = torch.rand(1, N, generator=torch.Generator().manual_seed(100 * ci + 70 + rank)) + 0.5
        output_shape = [*shape[:-1], N]
        out = ref._fused_scaled_matmul_reduce_scatter_fallback(
            A, B, A_scale, B_scale, c["op"], sd, sd, g, output_shape, None, None, BF16, False
        )
        rec.update(A=A, B_t=B.t().contiguous(), A_scale=A_scale, B_scale=B_scale, output_shape=output_shape, out=out.contiguous())
    return rec


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AUTOPARALLEL_REFERENCE", "")
    if not os.path.isdir(ref_root):
        raise SystemExit("usage: pass the AutoParallel source tree as the first argument (or in $AUTOPARALLEL_REFERENCE)")
    sys.path.insert(0, ref_root)
    import autoparallel.asynctp_ops as ref
    from torch.testing._internal.distributed.multi_threaded_pg import _install_threaded_pg, _uninstall_threaded_pg

    cases = _cases()
    results: dict[int, list] = {}
    errors: dict[int, str] = {}

    def run_group(which):
        store = dist.HashStore()

        def worker(rank):
            dist.init_process_group(backend="threaded", rank=rank, world_size=WORLD, store=store)
            g = dist.group.WORLD.group_name
            try:
                for ci, c in enumerate(cases):
                    if c["scaled_mm"] == which:
                        results.setdefault(rank, []).append(_run_case(ref, ci, c, rank, g))
            except BaseException:
                errors[rank] = traceback.format_exc()

        threads = [threading.Thread(target=worker, args=(r,)) for r in range(WORLD)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()

    torch._C._distributed_c10d._set_thread_isolation_mode(True)
    _install_threaded_pg()
    try:
        run_group("torch-cpu")
        # From here on aten::_scaled_mm on CPU is the row-wise stand-in (this process only).
        aten_cpu = torch.library.Library("aten", "IMPL")
        aten_cpu.impl("_scaled_mm", _scaled_mm_rowwise_cpu, "CPU")
        run_group("stand-in")
    finally:
        _uninstall_threaded_pg()
        torch._C._distributed_c10d._set_thread_isolation_mode(False)
    if errors:
        raise SystemExit("\n".join(errors.values()))
    per_rank = [results[r] for r in range(WORLD)]
    for r in per_rank:
        for rec in r:
            rec["out_dtypes"] = [str(d) for d in rec.get("out_dtypes", ())]
    torch.save(dict(world=WORLD, torch=torch.__version__, ranks=per_rank), OUT)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(per_rank[0])} cases)")


if __name__ == "__main__":
    main()
