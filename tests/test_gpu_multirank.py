"""Multi-rank parity on real GPUs (one process per GPU, NCCL for bootstrap only): the fused
kernels with their in-kernel NVLink exchange against the CPU oracle and against the golden
outputs of the reference's fallbacks. Skipped on machines with fewer than two GPUs."""
import pytest
import torch

from tests._mp import run_ranks

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
FP8_TOL = 3e-2


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, golden, golden_fp8):
    import torch.distributed as dist

    import autoparallel_b200.asynctp_ops  # noqa: F401
    from autoparallel_b200 import symm
    from oracle import asynctp_oracle as orc

    dev = torch.device("cuda", rank)
    g = dist.group.WORLD.group_name
    ns = torch.ops._ap_symm_mem

    def err(out, ref64_fn):
        """Relative Frobenius error against an fp64 reference computed on the device (the large cases would
        take minutes on the host cores)."""
        ref = ref64_fn()
        return ((out.double() - ref).norm() / ref.norm().clamp_min(1e-300)).item()

    def d64(t):
        return t.to(dev).double()

    # ---- golden fixtures (world 2 only): the reference's own outputs for these inputs
    if world == 2:
        mine, other = golden["ranks"][rank], golden["ranks"][1 - rank]
        for rec in mine:
            if rec["dtype"] != "torch.bfloat16":
                continue
            if rec["kind"] == "ag_mm":
                A_out, outs = ns.fused_all_gather_matmul(rec["A_shard"].to(dev), [b.to(dev) for b in rec["Bs"]], rec["gather_dim"], g)
                assert torch.equal(A_out.cpu(), rec["A_out"])
                for o, gold in zip(outs, rec["outs"]):
                    torch.testing.assert_close(o.cpu().float(), gold.float(), rtol=2 ** -7, atol=2e-3)
            elif rec["kind"] == "mm_rs":
                out = ns.fused_matmul_reduce_scatter(rec["A"].to(dev), rec["B"].to(dev), rec["op"], rec["scatter_dim"], g)
                assert out.shape == rec["out"].shape
                torch.testing.assert_close(out.cpu().float(), rec["out"].float(), rtol=2 ** -6, atol=4e-3)
        # ---- the reference's fp8 outputs (tests/golden/asynctp_golden_fp8.pt and the tensor-wise cases of the first
        #      fixture) through the CUDA path: every scale mode of the all-gather, bias, result scale, 3-D operands,
        #      both output types, reduce-scatter along dim 0 and 1. Same calls and tolerances as the CPU run of the
        #      host path (tests/test_host_end_to_end_cpu.py).
        dts = {"torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}

        def close(o, gold, rs=False):
            assert o.shape == gold.shape and o.dtype == gold.dtype, (o.shape, gold.shape, o.dtype, gold.dtype)
            if rs:   # the reference rounds every partial to bf16 before the sum, this path keeps its own in fp32
                torch.testing.assert_close(o.cpu().float(), gold.float(), rtol=2 ** -6, atol=max(4e-3, 2 ** -7 * float(gold.float().abs().max())))
            elif o.dtype == torch.float32:
                torch.testing.assert_close(o.cpu(), gold, rtol=1e-5, atol=1e-5)
            else:
                torch.testing.assert_close(o.cpu().float(), gold.float(), rtol=2 ** -7, atol=2e-3)

        n_fp8 = 0
        for rec in mine:
            if rec["kind"] == "smm_rs":
                out = ns.fused_scaled_matmul_reduce_scatter(
                    rec["A"].to(dev), rec["B_t"].to(dev).t(), rec["A_scale"].to(dev), rec["B_scale"].to(dev), rec["op"], 0, 0, g,
                    [rec["shape"][0], rec["N"]], None, None, torch.bfloat16, False)
                close(out, rec["out"], rs=True)
                n_fp8 += 1
        for rec in golden_fp8["ranks"][rank]:
            opt = lambda t: None if t is None else t.to(dev)   # noqa: E731
            if rec["kind"] == "sag_mm":
                Bs = [bt.to(dev).t() for bt in rec["Bs_t"]]
                A_out, outs = ns.fused_all_gather_scaled_matmul(
                    rec["A_shard"].to(dev), Bs, rec["A_scale"].to(dev), [s.to(dev) for s in rec["B_scales"]], rec["gather_dim"], g,
                    [opt(b) for b in rec["biases"]], [opt(r) for r in rec["result_scales"]], [dts[d] for d in rec["out_dtypes"]],
                    [False] * len(Bs))
                what = (rec["mode"], rec["shape"], rec["gather_dim"])
                assert A_out.shape == rec["A_out"].shape, what
                assert torch.equal(A_out.contiguous().cpu().view(torch.uint8), rec["A_out"].view(torch.uint8)), what
                for o, gold in zip(outs, rec["outs"]):
                    close(o, gold)
            else:
                out = ns.fused_scaled_matmul_reduce_scatter(
                    rec["A"].to(dev), rec["B_t"].to(dev).t(), rec["A_scale"].to(dev), rec["B_scale"].to(dev), rec["op"],
                    rec["scatter_dim"], rec["scatter_dim"], g, list(rec["output_shape"]), None, None, torch.bfloat16, False)
                close(out, rec["out"], rs=True)
            n_fp8 += 1
        assert n_fp8 == 2 + 12, n_fp8

    # ---- all-gather -> matmul against the oracle, ragged and multi-B shapes, both B layouts
    for rows, K, Ns, return_A, transposed in [
        (256, 256, [256], True, False),
        (1000, 520, [264, 128], False, True),
        (130, 72, [8], True, False),
        (2048, 4096, [1792, 1792], False, False),
        (512, 4096, [512, 128, 128], True, True),
    ]:
        shards = [orc.activations(r, rows, K) for r in range(world)]
        Bs = [orc.weights(7 + i, K, n) for i, n in enumerate(Ns)]
        dev_Bs = [b.to(dev).t().contiguous().t() if transposed else b.to(dev) for b in Bs]
        A_out, outs = ns.fused_all_gather_matmul(shards[rank].to(dev), dev_Bs, 0, g, return_A=return_A)
        A_ref, outs_ref = orc.all_gather_matmul_local(shards, Bs, 0, return_A)
        if return_A:
            assert torch.equal(A_out.cpu(), A_ref)
        A64 = d64(torch.cat(shards))
        for o, b in zip(outs, Bs):
            e = err(o, lambda: A64 @ d64(b))
            assert e <= BF16_TOL, (rows, K, Ns, e)
        del A64

    # ---- matmul -> reduce-scatter against the oracle
    for M, K, N, op in [(512, 256, 256, "sum"), (2000 // world * world, 520, 264, "avg"), (8192, 1792, 4096, "sum"), (128 * world, 64, 8, "sum")]:
        As = [orc.activations(20 + r, M, K) for r in range(world)]
        Ws = [orc.weights(30 + r, K, N) for r in range(world)]
        out = ns.fused_matmul_reduce_scatter(As[rank].to(dev), Ws[rank].to(dev), op, 0, g)
        lo, hi = rank * (M // world), (rank + 1) * (M // world)
        ref64 = sum(d64(a[lo:hi]) @ d64(w) for a, w in zip(As, Ws))
        if op == "avg":
            ref64 = ref64 / world
        assert out.shape == ref64.shape
        e = err(out, lambda: ref64)
        assert e <= BF16_TOL, (M, K, N, op, e)
        # never further from fp64 than the reference's decomposition (bf16 partials summed, autoparallel/asynctp_ops.py:1180-1185)
        parts = torch.stack([(a[lo:hi].to(dev) @ w.to(dev)).float() for a, w in zip(As, Ws)])
        oracle_out = (parts.sum(0) if op == "sum" else parts.mean(0)).bfloat16()
        assert e <= 1.5 * err(oracle_out, lambda: ref64) + 1e-4
        del ref64, parts

    # ---- 3-D operands, gather / scatter along dim 1
    sh3 = [orc.activations(40 + r, 4 * 32, 64).view(4, 32, 64) for r in range(world)]
    B = orc.weights(7, 64, 40)
    A_out, (o,) = ns.fused_all_gather_matmul(sh3[rank].to(dev), [B.to(dev)], 1, g)
    A_ref, (o_ref,) = orc.all_gather_matmul_local(sh3, [B], 1)
    assert torch.equal(A_out.cpu(), A_ref) and orc.rel_fro_error(o, o_ref.double()) <= BF16_TOL
    X3 = [orc.activations(50 + r, 4 * 32 * world, 64).view(4, 32 * world, 64) for r in range(world)]
    out = ns.fused_matmul_reduce_scatter(X3[rank].to(dev), B.to(dev), "sum", 1, g)
    ref = orc.matmul_reduce_scatter_local(X3, [B] * world, "sum", 1)[rank]
    assert out.shape == ref.shape and orc.rel_fro_error(out, ref.double()) <= BF16_TOL

    # ---- gather / scatter along the LAST dim (K-split accumulation, column-split reduce-scatter)
    ksh = [orc.activations(90 + r, 6 * 50, 192).view(6, 50, 192) for r in range(world)]
    Bk = [orc.weights(91, 192 * world, 264), orc.weights(92, 192 * world, 512)]
    A_out, outs = ns.fused_all_gather_matmul(ksh[rank].to(dev), [b.to(dev) for b in Bk], 2, g)
    A_ref, outs_ref = orc.all_gather_matmul_local(ksh, Bk, 2)
    assert torch.equal(A_out.cpu(), A_ref)
    for o, b in zip(outs, Bk):
        assert o.shape == (6, 50, b.shape[1])
        assert orc.rel_fro_error(o, torch.cat(ksh, dim=-1).double() @ b.double()) <= BF16_TOL
    Xc = [orc.activations(93 + r, 4 * 130, 192).view(4, 130, 192) for r in range(world)]
    Wc = [orc.weights(94 + r, 192, 256 * world) for r in range(world)]
    out = ns.fused_matmul_reduce_scatter(Xc[rank].to(dev), Wc[rank].to(dev), "avg", 2, g)
    ref64 = (sum(x.double() @ w.double() for x, w in zip(Xc, Wc)) / world).chunk(world, dim=-1)[rank]
    assert out.shape == ref64.shape and orc.rel_fro_error(out, ref64) <= BF16_TOL

    # ---- fp8 row-wise, both ops, sharded and replicated row scales
    rows, K, N = 384, 512, 264
    xs = [orc.quantize_rowwise(orc.activations(60 + r, rows, K, torch.float32), 1) for r in range(world)]
    w8, sw = orc.quantize_rowwise(orc.weights(70, K, N, torch.float32), 0)
    w_dev = w8.to(dev).t().contiguous().t()
    bias = orc.weights(71, 1, N, torch.bfloat16, std=1.0).view(-1)
    A_ref, (o_ref,) = orc.all_gather_scaled_matmul_local(
        [x[0] for x in xs], [w8], [x[1] for x in xs], [sw], 0, [bias], [None], [torch.bfloat16], compute_dtype=torch.float64
    )
    A_out, (o,) = ns.fused_all_gather_scaled_matmul(
        xs[rank][0].to(dev), [w_dev], xs[rank][1].to(dev), [sw.to(dev)], 0, g, [bias.to(dev)], [None], [torch.bfloat16], [False]
    )
    assert torch.equal(A_out.cpu().view(torch.uint8), A_ref.view(torch.uint8))
    assert orc.rel_fro_error(o, o_ref.double()) <= FP8_TOL
    full_scale = torch.cat([x[1] for x in xs])
    _, (o2,) = ns.fused_all_gather_scaled_matmul(
        xs[rank][0].to(dev), [w_dev], full_scale.to(dev), [sw.to(dev)], 0, g, [bias.to(dev)], [None], [torch.bfloat16], [False]
    )
    assert torch.equal(o, o2)
    Mrs = 256 * world
    ys = [orc.quantize_rowwise(orc.activations(80 + r, Mrs, K, torch.float32), 1) for r in range(world)]
    out = ns.fused_scaled_matmul_reduce_scatter(
        ys[rank][0].to(dev), w_dev, ys[rank][1].to(dev), sw.to(dev), "sum", 0, 0, g, [Mrs, N], None, None, torch.bfloat16, False
    )
    ref = orc.scaled_matmul_reduce_scatter_local(
        [y[0] for y in ys], [w8] * world, [y[1] for y in ys], [sw] * world, "sum", 0, [Mrs, N], out_dtype=torch.float32,
        compute_dtype=torch.float64,
    )[rank]
    assert out.shape == ref.shape and orc.rel_fro_error(out, ref.double()) <= FP8_TOL

    # ---- float16 operands: the all-gather as is, the reduce-scatter with fp32 partials rounded once at the end
    hs = [orc.activations(130 + r, 384, 520, torch.float16) for r in range(world)]
    Bh = orc.weights(131, 520, 264, torch.float16, std=0.05)
    A_out, (o,) = ns.fused_all_gather_matmul(hs[rank].to(dev), [Bh.to(dev)], 0, g)
    assert o.dtype == torch.float16 and torch.equal(A_out.cpu(), torch.cat(hs))
    assert err(o, lambda: d64(torch.cat(hs)) @ d64(Bh)) <= BF16_TOL / 4
    Xh = [orc.activations(140 + r, 256 * world, 520, torch.float16) for r in range(world)]
    out = ns.fused_matmul_reduce_scatter(Xh[rank].to(dev), Bh.to(dev), "sum", 0, g)
    lo, hi = rank * 256, (rank + 1) * 256
    assert out.dtype == torch.float16 and out.shape == (256, 264)
    assert err(out, lambda: sum(d64(x[lo:hi]) for x in Xh) @ d64(Bh)) <= BF16_TOL / 4

    # ---- stand-alone collectives over the same arena and flags
    x = orc.activations(110 + rank, 300, 264).to(dev)
    got = ns._low_contention_all_gather(x, g)
    want = torch.cat([orc.activations(110 + r, 300, 264) for r in range(world)])
    assert torch.equal(got.cpu(), want)
    for dt, tol in ((torch.bfloat16, 1e-2), (torch.float32, 1e-6)):
        ys = [orc.activations(120 + r, 64 * world, 200, dt) for r in range(world)]
        for op in ("sum", "avg"):
            got = ns._low_contention_reduce_scatter(ys[rank].to(dev), op, g)
            want = sum(y.double() for y in ys).chunk(world)[rank] / (world if op == "avg" else 1)
            assert got.shape == want.shape and got.dtype == dt and orc.rel_fro_error(got, want) <= tol

    # ---- many back-to-back calls: the two halves of the arena and the epoch flags hold up
    A = orc.activations(rank, 1024, 1024).to(dev)
    W = orc.weights(7, 1024, 512).to(dev)
    first = None
    for _ in range(12):
        _, (o,) = ns.fused_all_gather_matmul(A, [W], 0, g, return_A=False)
        r = ns.fused_matmul_reduce_scatter(o, W.t().contiguous(), "sum", 0, g)
        if first is None:
            first = (o.clone(), r.clone())
        else:
            assert torch.equal(o, first[0]) and torch.equal(r, first[1])
    torch.cuda.synchronize()
    symm.sync_check()
    symm.shutdown()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ops_multirank(world, golden, golden_fp8):
    if _ngpus() < world:
        pytest.skip(f"needs {world} GPUs")
    from autoparallel_b200.build import build_native

    build_native()
    run_ranks(_worker, world, golden, golden_fp8, backend="nccl")
