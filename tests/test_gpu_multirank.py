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


def _worker(rank, world, golden):
    import torch.distributed as dist

    import autoparallel_b200.asynctp_ops  # noqa: F401
    from autoparallel_b200 import symm
    from oracle import asynctp_oracle as orc

    dev = torch.device("cuda", rank)
    g = dist.group.WORLD.group_name
    ns = torch.ops._ap_symm_mem

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
        for o, b in zip(outs, Bs):
            err = orc.rel_fro_error(o, torch.cat(shards).double() @ b.double())
            assert err <= BF16_TOL, (rows, K, Ns, err)

    # ---- matmul -> reduce-scatter against the oracle
    for M, K, N, op in [(512, 256, 256, "sum"), (2000 // world * world, 520, 264, "avg"), (8192, 1792, 4096, "sum"), (128 * world, 64, 8, "sum")]:
        As = [orc.activations(20 + r, M, K) for r in range(world)]
        Ws = [orc.weights(30 + r, K, N) for r in range(world)]
        out = ns.fused_matmul_reduce_scatter(As[rank].to(dev), Ws[rank].to(dev), op, 0, g)
        ref64 = sum(a.double() @ w.double() for a, w in zip(As, Ws))
        if op == "avg":
            ref64 = ref64 / world
        ref64 = ref64.chunk(world)[rank]
        assert out.shape == ref64.shape
        err = orc.rel_fro_error(out, ref64)
        assert err <= BF16_TOL, (M, K, N, op, err)
        oracle_out = orc.matmul_reduce_scatter_local(As, Ws, op, 0)[rank]
        assert err <= 1.5 * orc.rel_fro_error(oracle_out, ref64) + 1e-4

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
def test_fused_ops_multirank(world, golden):
    if _ngpus() < world:
        pytest.skip(f"needs {world} GPUs")
    from autoparallel_b200.build import build_native

    build_native()
    run_ranks(_worker, world, golden, backend="nccl")
