"""The host path end to end on CPU, two gloo ranks, against the REFERENCE's outputs.

The CUDA library is replaced by ``tests/_abi_model.ModelLib``, which executes the argument
structs the host code builds exactly as include/apk.h documents them. Everything above the C ABI
is the shipped code: argument checks, moving the gather / scatter dimension to the front,
flattening and un-flattening, scale-mode handling, ``output_shape``, workspace creation and
growth over the process group, epochs. The results are compared with what the reference's own
fallbacks produced for the same inputs (tests/golden/, both fixtures), so a wrong stride, a
swapped dimension or a mis-marshalled scale shows up without a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from tests._mp import run_ranks

_DT = {"torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}


def _install_model():
    import ctypes as C

    import autoparallel_b200.asynctp_ops as ops
    from autoparallel_b200 import _native as nat
    from autoparallel_b200 import symm
    from tests._abi_model import ModelLib

    model = ModelLib()
    nat.lib = lambda: model
    ops._stream_ptr = lambda device: C.c_void_p(0)
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.is_current_stream_capturing = lambda: False

    class _NoDevice:
        def __init__(self, *a):
            pass

        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    torch.cuda.device = _NoDevice
    return ops, symm, model


def _close(o, g, rtol=2 ** -7, atol=2e-3):
    assert o.shape == g.shape and o.dtype == g.dtype, (o.shape, g.shape, o.dtype, g.dtype)
    if o.dtype == torch.float32:
        torch.testing.assert_close(o, g, rtol=1e-5, atol=1e-5)
    else:
        torch.testing.assert_close(o.float(), g.float(), rtol=rtol, atol=atol)


def _close_rs(o, g):
    """Reduce-scatter outputs. The reference rounds every rank's partial to bf16 before the sum,
    this path keeps the local partial in fp32: results differ by up to half a bf16 ulp OF A
    PARTIAL, which can exceed an ulp of a small (cancelled) sum, hence the norm-scaled atol."""
    _close(o, g, rtol=2 ** -6, atol=max(4e-3, 2 ** -7 * float(g.float().abs().max())))


def _worker(rank, world, golden, golden_fp8):
    ops, symm, model = _install_model()
    g = dist.group.WORLD.group_name
    mine = golden["ranks"][rank]
    n_checked = 0

    # ---- bf16: all-gather -> matmul (every gather dim, the last one included) and matmul -> reduce-scatter
    for rec in mine:
        if rec["dtype"] != "torch.bfloat16":
            continue      # the fused ops take bf16 / fp8 only; fp32 cases pin the oracle
        if rec["kind"] == "ag_mm":
            A_out, outs = ops._fused_all_gather_matmul(rec["A_shard"], rec["Bs"], rec["gather_dim"], g, return_A=True)
            assert A_out.shape == rec["A_out"].shape and torch.equal(A_out, rec["A_out"]), (rec["shape"], rec["gather_dim"])
            for o, gold in zip(outs, rec["outs"]):
                _close(o, gold)
            A_none, outs2 = ops._fused_all_gather_matmul(rec["A_shard"], rec["Bs"], rec["gather_dim"], g, return_A=False)
            assert A_none is None and all(torch.equal(x, y) for x, y in zip(outs, outs2))
            n_checked += 1
        elif rec["kind"] == "mm_rs":
            out = ops._fused_matmul_reduce_scatter(rec["A"], rec["B"], rec["op"], rec["scatter_dim"], g)
            _close_rs(out, rec["out"])
            n_checked += 1
    # non-contiguous input and a transposed-view B take the no-copy paths and give the same result
    rec = next(r for r in mine if r["kind"] == "ag_mm" and r["dtype"] == "torch.bfloat16" and r["gather_dim"] == 1)
    A_nc = rec["A_shard"].transpose(0, 1).contiguous().transpose(0, 1)
    Bs_t = [b.t().contiguous().t() for b in rec["Bs"]]
    A_out, outs = ops._fused_all_gather_matmul(A_nc, Bs_t, 1, g)
    assert torch.equal(A_out, rec["A_out"])
    for o, gold in zip(outs, rec["outs"]):
        _close(o, gold)

    # ---- fp8, tensor-wise scaled matmul -> reduce-scatter (first fixture)
    for rec in mine:
        if rec["kind"] == "smm_rs":
            out = ops._fused_scaled_matmul_reduce_scatter(
                rec["A"], rec["B_t"].t(), rec["A_scale"], rec["B_scale"], rec["op"], 0, 0, g,
                [rec["shape"][0], rec["N"]], None, None, torch.bfloat16, False,
            )
            _close_rs(out, rec["out"])
            n_checked += 1

    # ---- fp8 fixture: every scale mode of the all-gather, bias, result scale, 3-D, both output types
    for rec in golden_fp8["ranks"][rank]:
        if rec["kind"] == "sag_mm":
            Bs = [bt.t() for bt in rec["Bs_t"]]
            A_out, outs = ops._fused_all_gather_scaled_matmul(
                rec["A_shard"], Bs, rec["A_scale"], rec["B_scales"], rec["gather_dim"], g, rec["biases"],
                rec["result_scales"], [_DT[d] for d in rec["out_dtypes"]], [False] * len(Bs),
            )
            what = (rec["mode"], rec["shape"], rec["gather_dim"])
            assert A_out.shape == rec["A_out"].shape, what
            assert torch.equal(A_out.contiguous().view(torch.uint8), rec["A_out"].view(torch.uint8)), what
            for o, gold in zip(outs, rec["outs"]):
                _close(o, gold)
        else:
            out = ops._fused_scaled_matmul_reduce_scatter(
                rec["A"], rec["B_t"].t(), rec["A_scale"], rec["B_scale"], rec["op"], rec["scatter_dim"], rec["scatter_dim"], g,
                list(rec["output_shape"]), None, None, torch.bfloat16, False,
            )
            _close_rs(out, rec["out"])
        n_checked += 1

    # ---- a scatter dim folded into the rows by a pre-matmul reshape (orig 1 -> 0 after), batch 2: like the
    #      reference's CUDA body (autoparallel/asynctp_ops.py:1375-1423) the result is row chunk `rank` of the
    #      flattened [B*S, N] product, viewed as [B, S/world, N]
    from oracle import asynctp_oracle as orc

    Bt, S, K, N = 2, 8, 32, 16
    xs = [orc.quantize_rowwise(orc.activations(200 + r, Bt * S, K, torch.float32), 1) for r in range(world)]
    w8, sw = orc.quantize_rowwise(orc.weights(210, K, N, torch.float32, std=0.5), 0)
    out = ops._fused_scaled_matmul_reduce_scatter(
        xs[rank][0], w8.t().contiguous().t(), xs[rank][1], sw, "sum", 1, 0, g, [Bt, S, N], None, None, torch.bfloat16, False
    )
    flat = orc.scaled_matmul_reduce_scatter_local(
        [x[0] for x in xs], [w8] * world, [x[1] for x in xs], [sw] * world, "sum", 0, [Bt * S, N], out_dtype=torch.bfloat16
    )[rank]
    assert out.shape == (Bt, S // world, N)
    _close_rs(out, flat.view(Bt, S // world, N))

    # ---- the stand-alone collectives' host side
    x = torch.arange(rank * 100, rank * 100 + 24 * 8, dtype=torch.float32).view(24, 8)
    got = ops._low_contention_all_gather(x, g)
    want = torch.cat([torch.arange(r * 100, r * 100 + 24 * 8, dtype=torch.float32).view(24, 8) for r in range(world)])
    assert torch.equal(got, want)
    y = torch.full((8 * world, 16), float(rank + 1), dtype=torch.bfloat16)
    got = ops._low_contention_reduce_scatter(y, "avg", g)
    assert got.shape == (8, 16) and torch.equal(got.float(), torch.full((8, 16), (1 + world) / 2))

    assert n_checked == 4 + 6 + 2 + 12, n_checked
    assert model.calls.count("ag_gemm") >= 16 and model.calls.count("gemm_rs") >= 11
    # one collective per call: every rank's epoch advanced in lock step
    epochs = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(epochs, torch.tensor([symm.get_workspace(g, torch.device("cpu")).epoch]))
    assert len({int(e) for e in epochs}) == 1 and int(epochs[0]) > 0
    symm.shutdown()
    assert not model.live


def test_host_path_matches_reference_outputs_on_cpu(golden, golden_fp8):
    run_ranks(_worker, 2, golden, golden_fp8)
