"""Parity of the sm_100a kernels on one GPU (a tensor-parallel group of one rank), called through
torch.ops._ap_symm_mem -> ctypes -> the C ABI, checked against the CPU oracle and the golden
fixtures. Tolerances are the ones the task states: relative Frobenius error <= 1e-2 for bf16
with fp32 accumulation and <= 3e-2 for fp8, against an fp64 product of the same (already
quantised) operands."""
import ctypes as C
import os
import tempfile

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
FP8_TOL = 3e-2


@pytest.fixture(scope="module")
def group():
    from autoparallel_b200.build import build_native
    import autoparallel_b200.asynctp_ops  # noqa: F401  registers the ops
    from autoparallel_b200 import symm

    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    build_native()
    torch.cuda.set_device(0)
    if dist.is_initialized():
        dist.destroy_process_group()
    with tempfile.TemporaryDirectory() as d:
        dist.init_process_group("gloo", init_method=f"file://{os.path.join(d, 'init')}", rank=0, world_size=1)
        yield dist.group.WORLD.group_name
        torch.cuda.synchronize()
        symm.sync_check()
        symm.shutdown()
        dist.destroy_process_group()


def _orc():
    from oracle import asynctp_oracle as orc

    return orc


def _ag(A, Bs, gd, g, return_A=True):
    A_out, outs = torch.ops._ap_symm_mem.fused_all_gather_matmul(A.cuda(), [b.cuda() for b in Bs], gd, g, return_A=return_A)
    torch.cuda.synchronize()
    return A_out, outs


@pytest.mark.parametrize(
    "rows,K,Ns",
    [(128, 64, [256]), (1, 8, [8]), (127, 72, [8, 16]), (1000, 1032, [264, 128]), (384, 4096, [1792, 1792]),
     (512, 512, [64, 128, 32]), (300, 200, [512, 128, 128, 40])],
)
@pytest.mark.parametrize("b_layout", ["row_major", "transposed_view"])
def test_all_gather_matmul_shapes(group, rows, K, Ns, b_layout):
    orc = _orc()
    A = orc.activations(0, rows, K)
    Bs = [orc.weights(7 + i, K, n) for i, n in enumerate(Ns)]
    dev_Bs = [b.cuda() if b_layout == "row_major" else b.cuda().t().contiguous().t() for b in Bs]
    A_out, outs = torch.ops._ap_symm_mem.fused_all_gather_matmul(A.cuda(), dev_Bs, 0, group)
    torch.cuda.synchronize()
    A_ref, outs_ref = orc.all_gather_matmul_local([A], Bs, 0)
    assert torch.equal(A_out.cpu(), A_ref)
    for o, o_ref, b in zip(outs, outs_ref, Bs):
        assert o.shape == o_ref.shape and o.dtype == o_ref.dtype
        assert not torch.isnan(o).any()
        ref64 = A.double() @ b.double()
        assert orc.rel_fro_error(o, ref64) <= BF16_TOL
        # and as close to fp64 as the reference decomposition itself (bf16 output rounding)
        assert orc.rel_fro_error(o, ref64) <= 1.5 * orc.rel_fro_error(o_ref, ref64) + 1e-4


def test_all_gather_matmul_nd_and_return_A(group):
    orc = _orc()
    A = orc.activations(3, 4 * 6, 64).view(4, 6, 64)
    Bs = [orc.weights(7, 64, 40), orc.weights(8, 64, 24)]
    for gd in (0, 1):
        for return_A in (True, False):
            A_out, outs = _ag(A, Bs, gd, group, return_A)
            A_ref, outs_ref = orc.all_gather_matmul_local([A], Bs, gd, return_A)
            assert (A_out is None) == (not return_A)
            if return_A:
                assert torch.equal(A_out.cpu(), A_ref)
            for o, o_ref in zip(outs, outs_ref):
                assert o.shape == o_ref.shape
                assert orc.rel_fro_error(o, o_ref.double()) <= BF16_TOL
    # a strided A (gather_dim not in front in memory) is accepted, like the reference
    A_nc = A.transpose(0, 1).contiguous().transpose(0, 1)
    _, outs = _ag(A_nc, Bs, 0, group)
    _, outs_ref = orc.all_gather_matmul_local([A], Bs, 0)
    assert orc.rel_fro_error(outs[0], outs_ref[0].double()) <= BF16_TOL


def test_last_dim_variants_single_rank(group):
    """Gather / scatter along the last dim with a group of one: the K-split and column-split paths."""
    orc = _orc()
    A = orc.activations(4, 6 * 50, 192).view(6, 50, 192)
    Bs = [orc.weights(7, 192, 264), orc.weights(8, 192, 128)]
    A_out, outs = _ag(A, Bs, 2, group, True)
    A_ref, outs_ref = orc.all_gather_matmul_local([A], Bs, 2, True)
    assert torch.equal(A_out.cpu(), A_ref)
    for o, o_ref, b in zip(outs, outs_ref, Bs):
        assert o.shape == o_ref.shape and orc.rel_fro_error(o, A.double() @ b.double()) <= BF16_TOL
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(A.cuda(), Bs[0].cuda(), "sum", 2, group)
    (ref,) = orc.matmul_reduce_scatter_local([A], [Bs[0]], "sum", 2)
    assert out.shape == ref.shape and orc.rel_fro_error(out, A.double() @ Bs[0].double()) <= BF16_TOL


def test_all_gather_last_dim_receive_side_on_one_gpu(group):
    """Rank 0 of a two-rank all-gather along the LAST dim on a single GPU (the peer's K-slice is staged
    beforehand): out = A_0 @ B[:K] + A_1 @ B[K:], accumulated in TMEM in arrival order."""
    from autoparallel_b200 import _native as nat
    from tests.test_zz_no_alloc import _TwoRankHarness

    L = nat.lib()
    orc = _orc()
    rows, Kc, N = 384, 256, 264
    h = _TwoRankHarness(nat, rows, Kc, False)
    B = orc.weights(7, 2 * Kc, N).cuda()
    ref64 = torch.cat([s.cpu().double() for s in h.shards], dim=1) @ B.cpu().double()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for epoch in (1, 2):
        out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        stacked = torch.empty(2 * rows, Kc, dtype=torch.bfloat16, device="cuda")
        c = h.comm(epoch, with_ctrl=True)
        a = nat.ApkAgGemmArgs()
        a.dtype, a.rows_per_rank, a.K, a.nB, a.gather_k = nat.APK_BF16, rows, Kc, 1, 1
        a.A_shard, a.lda = h.shards[0].data_ptr(), Kc
        a.A_gathered, a.return_A = stacked.data_ptr(), 1
        op = a.Bs[0]
        op.B, op.ldb, op.n_major, op.N = B.data_ptr(), N, 1, N
        op.out, op.ldo, op.out_dtype = out.data_ptr(), N, nat.APK_BF16
        assert L.apk_ag_gemm(C.byref(c), C.byref(a), stream) == nat.APK_OK, L.apk_last_error()
        raw = C.c_uint32(0)
        assert L.apk_check_status(C.byref(c), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()
        assert orc.rel_fro_error(out, ref64) <= BF16_TOL
        assert torch.equal(stacked[:rows], h.shards[0]) and torch.equal(stacked[rows:], h.shards[1])


def test_stand_alone_collectives_single_rank(group):
    x = torch.randn(37, 24, device="cuda").bfloat16()
    assert torch.equal(torch.ops._ap_symm_mem._low_contention_all_gather(x, group), x)
    y = torch.randn(16, 8, device="cuda")
    torch.testing.assert_close(torch.ops._ap_symm_mem._low_contention_reduce_scatter(y, "avg", group), y)
    with pytest.raises(ValueError, match="reduce_op must be sum or avg"):
        torch.ops._ap_symm_mem._low_contention_reduce_scatter(y, "max", group)


def test_stand_alone_collectives_receive_side_on_one_gpu(group):
    """Rank 0 of a 4-rank all-gather and reduce-scatter on one GPU: the peers' staged shards / partial
    parts and their flags are placed beforehand, so the pull, the pushes and the fp32 sum all run."""
    from autoparallel_b200 import _native as nat

    L = nat.lib()
    world, nbytes = 4, 300 * 264 * 2
    shards = [torch.randn(300, 264, device="cuda").bfloat16() for _ in range(world)]
    half = ((world * nbytes + 4095) // 4096) * 4096
    arenas = [torch.zeros(2 * half, dtype=torch.uint8, device="cuda") for _ in range(world)]
    pads = [torch.zeros(1 << 17, dtype=torch.int32, device="cuda") for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctrl = torch.zeros(1024, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def comm(epoch):
        c = nat.ApkComm()
        c.rank, c.world = 0, world
        for r in range(world):
            c.data[r], c.flags[r] = arenas[r].data_ptr(), pads[r].data_ptr()
        c.data_bytes, c.flag_bytes = 2 * half, pads[0].numel() * 4
        c.ctrl, c.ctrl_bytes = ctrl.data_ptr(), ctrl.numel() * 4
        c.status, c.epoch, c.timeout_s = status.data_ptr(), epoch, 5.0
        return c

    raw = C.c_uint32(0)
    # all-gather: peers r staged their shard at the start of their arena half; "staged" flags live 32 words apart
    for r in range(1, world):
        for h in range(2):
            arenas[r][h * half: h * half + nbytes] = shards[r].view(torch.uint8).view(-1)
        pads[0][r * 32] = 1000
    for epoch in (1, 2):
        out = torch.zeros(world * 300, 264, dtype=torch.bfloat16, device="cuda")
        c = comm(epoch)
        assert L.apk_all_gather(C.byref(c), C.c_void_p(shards[0].data_ptr()), C.c_void_p(out.data_ptr()), nbytes, stream) == 0, L.apk_last_error()
        assert L.apk_check_status(C.byref(c), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()
        assert torch.equal(out, torch.cat(shards))
        assert int(pads[2][0]) == epoch        # rank 0 told rank 2 that its shard is staged
    # reduce-scatter: peers' parts for rank 0 wait in slots 1..3 of rank 0's arena half, flags (source, tile 0) raised
    full = [torch.randn(world * 300, 264, device="cuda").bfloat16() for _ in range(world)]
    max_tiles = (pads[0].numel() * 4 - 4096) // 4 // world
    for r in range(1, world):
        for h in range(2):
            arenas[0][h * half + r * nbytes: h * half + (r + 1) * nbytes] = full[r][:300].contiguous().view(torch.uint8).view(-1)
        pads[0][1024 + r * max_tiles] = 1000
    want = sum(f[:300].double() for f in full) / world
    for epoch in (3, 4):
        out = torch.zeros(300, 264, dtype=torch.bfloat16, device="cuda")
        c = comm(epoch)
        assert L.apk_reduce_scatter(C.byref(c), C.c_void_p(full[0].data_ptr()), C.c_void_p(out.data_ptr()), nbytes,
                                    nat.APK_BF16, nat.APK_REDUCE_AVG, stream) == 0, L.apk_last_error()
        assert L.apk_check_status(C.byref(c), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()
        assert _orc().rel_fro_error(out, want.cpu()) <= BF16_TOL
        off = (epoch & 1) * half
        sent = arenas[2][off: off + nbytes].view(torch.bfloat16).view(300, 264)      # slot 0 of rank 2's arena
        assert torch.equal(sent, full[0][600:900])
        assert int(pads[2][1024]) == epoch


def test_golden_all_gather_matmul(group, golden):
    """bf16 golden cases: the gathered A the reference produced, times the Bs, must give its outputs."""
    orc = _orc()
    n = 0
    for rec in golden["ranks"][0]:
        if rec["kind"] != "ag_mm" or rec["dtype"] != "torch.bfloat16" or rec["gather_dim"] == len(rec["shape"]) - 1:
            continue
        gd = rec["gather_dim"]
        _, outs = _ag(rec["A_out"], rec["Bs"], gd, group, return_A=False)
        for o, gold in zip(outs, rec["outs"]):
            assert o.shape == gold.shape
            torch.testing.assert_close(o.cpu().float(), gold.float(), rtol=2 ** -7, atol=2e-3)
        n += 1
    assert n == 3


def test_golden_matmul_reduce_scatter_partials(group, golden):
    """Each rank's partial comes from the kernel (group of one); summed like the reference they give its output."""
    r0, r1 = golden["ranks"]
    n = 0
    for c0, c1 in zip(r0, r1):
        if c0["kind"] != "mm_rs" or c0["dtype"] != "torch.bfloat16" or c0["scatter_dim"] != 0:
            continue
        parts = [
            torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(c["A"].cuda(), c["B"].cuda(), "sum", 0, group).float().cpu()
            for c in (c0, c1)
        ]
        total = parts[0] + parts[1]
        if c0["op"] == "avg":
            total = total / 2
        for rank, c in enumerate((c0, c1)):
            mine = total.chunk(2, dim=0)[rank]
            torch.testing.assert_close(mine, c["out"].float(), rtol=2 ** -6, atol=4e-3)
        n += 1
    assert n == 4


@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (1000, 520, 264), (2048, 1792, 4096), (64, 128, 8)])
@pytest.mark.parametrize("op", ["sum", "avg"])
def test_matmul_reduce_scatter_single_rank(group, M, K, N, op):
    orc = _orc()
    A, B = orc.activations(1, M, K), orc.weights(9, K, N)
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(A.cuda(), B.cuda(), op, 0, group)
    torch.cuda.synchronize()
    (ref,) = orc.matmul_reduce_scatter_local([A], [B], op, 0)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert orc.rel_fro_error(out, A.double() @ B.double()) <= BF16_TOL


def test_matmul_reduce_scatter_3d(group):
    orc = _orc()
    A = orc.activations(2, 4 * 6, 64).view(4, 6, 64)
    B = orc.weights(9, 64, 40)
    for sd in (0, 1):
        out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(A.cuda(), B.cuda(), "sum", sd, group)
        (ref,) = orc.matmul_reduce_scatter_local([A], [B], "sum", sd)
        assert out.shape == ref.shape
        assert orc.rel_fro_error(out, (A.double() @ B.double())) <= BF16_TOL


def test_empty_and_errors(group):
    bf = torch.bfloat16
    A = torch.empty(0, 64, dtype=bf, device="cuda")
    B = torch.zeros(64, 16, dtype=bf, device="cuda")
    A_out, (o,) = torch.ops._ap_symm_mem.fused_all_gather_matmul(A, [B], 0, group)
    assert A_out.shape == (0, 64) and o.shape == (0, 16)
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(A, B, "sum", 0, group)
    assert out.shape == (0, 16)
    X = torch.zeros(8, 64, dtype=bf, device="cuda")
    with pytest.raises(ValueError, match="reduce_op must be sum or avg"):
        torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(X, B, "max", 0, group)
    with pytest.raises(ValueError, match="Invalid gather_dim"):
        torch.ops._ap_symm_mem.fused_all_gather_matmul(X, [B], 3, group)
    with pytest.raises(NotImplementedError, match="bfloat16, float16 or float8_e4m3fn"):
        torch.ops._ap_symm_mem.fused_all_gather_matmul(X.float(), [B.float()], 0, group)
    from autoparallel_b200._native import ApkError

    with pytest.raises(ApkError, match="multiple of"):  # N = 12 cannot be stored in 16-byte vectors
        torch.ops._ap_symm_mem.fused_all_gather_matmul(X, [torch.zeros(64, 12, dtype=bf, device="cuda")], 0, group)


# --------------------------------------------------------------------------------------- fp8
def _fp8_case(orc, rows, K, N, seed=0):
    x = orc.activations(seed, rows, K, torch.float32)
    w = orc.weights(seed + 7, K, N, torch.float32)
    a8, sa = orc.quantize_rowwise(x, 1)
    b8, sb = orc.quantize_rowwise(w, 0)
    return a8, sa, b8, sb


@pytest.mark.parametrize("rows,K,N", [(128, 128, 256), (1000, 1040, 264), (2048, 8192, 3584), (5, 16, 8)])
def test_scaled_all_gather_matmul_rowwise(group, rows, K, N):
    orc = _orc()
    a8, sa, b8, sb = _fp8_case(orc, rows, K, N)
    b_dev = b8.cuda().t().contiguous().t()  # column-major, as _scaled_mm requires
    A_out, (o,) = torch.ops._ap_symm_mem.fused_all_gather_scaled_matmul(
        a8.cuda(), [b_dev], sa.cuda(), [sb.cuda()], 0, group, [None], [None], [torch.bfloat16], [False]
    )
    torch.cuda.synchronize()
    assert torch.equal(A_out.cpu().view(torch.uint8), a8.view(torch.uint8))
    ref64 = (a8.double() * sa.double()) @ (b8.double() * sb.double())
    assert o.dtype == torch.bfloat16 and orc.rel_fro_error(o, ref64) <= FP8_TOL
    _, (o_ref,) = orc.all_gather_scaled_matmul_local([a8], [b8], [sa], [sb], 0, [None], [None], [torch.bfloat16])
    torch.testing.assert_close(o.cpu().float(), o_ref.float(), rtol=2 ** -7, atol=1e-3)
    # the oracle's restatement of row-wise scaling agrees with torch._scaled_mm on this GPU
    if K % 16 == 0 and N % 16 == 0:
        lib_out = torch._scaled_mm(a8.cuda(), b_dev, sa.cuda(), sb.cuda(), out_dtype=torch.bfloat16)
        torch.testing.assert_close(lib_out.cpu().float(), o_ref.float(), rtol=2 ** -6, atol=2e-3)


def test_scaled_all_gather_matmul_scale_modes_bias_result_scale(group):
    orc = _orc()
    a8, sa, b8, sb = _fp8_case(orc, 256, 256, 128, seed=3)
    b_dev = b8.cuda().t().contiguous().t()
    bias = orc.weights(99, 1, 128, torch.bfloat16, std=1.0).view(-1)
    rs = torch.tensor(0.5)
    t = torch.tensor(0.25)
    for a_scale in (sa, t):
        for out_dtype in (torch.bfloat16, torch.float32):
            _, (o,) = torch.ops._ap_symm_mem.fused_all_gather_scaled_matmul(
                a8.cuda(), [b_dev], a_scale.cuda(), [sb.cuda()], 0, group, [bias.cuda()], [rs.cuda()], [out_dtype], [True]
            )
            _, (o_ref,) = orc.all_gather_scaled_matmul_local(
                [a8], [b8], [a_scale], [sb], 0, [bias], [rs], [out_dtype], compute_dtype=torch.float64
            )
            assert o.dtype == out_dtype
            assert orc.rel_fro_error(o, o_ref.double()) <= (FP8_TOL if out_dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("op", ["sum", "avg"])
def test_scaled_matmul_reduce_scatter_single_rank(group, op):
    orc = _orc()
    a8, sa, b8, sb = _fp8_case(orc, 512, 384, 264, seed=5)
    b_dev = b8.cuda().t().contiguous().t()
    out = torch.ops._ap_symm_mem.fused_scaled_matmul_reduce_scatter(
        a8.cuda(), b_dev, sa.cuda(), sb.cuda(), op, 0, 0, group, [512, 264], None, None, torch.bfloat16, False
    )
    (ref,) = orc.scaled_matmul_reduce_scatter_local([a8], [b8], [sa], [sb], op, 0, [512, 264], out_dtype=torch.bfloat16)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    ref64 = (a8.double() * sa.double()) @ (b8.double() * sb.double())
    assert orc.rel_fro_error(out, ref64) <= FP8_TOL


# --------------------------------------------------------------------------------------- full size
def _freivalds(out, A, B, tol):
    """C x == A (B x) for random x, in fp64 on the device: an O(MN) check of a product of any size."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(out.shape[1], 4, device="cuda", dtype=torch.float64, generator=g)
    lhs = out.double() @ x
    rhs = A.double() @ (B.double() @ x)
    err = ((lhs - rhs).norm() / rhs.norm()).item()
    assert err <= tol, err


def test_full_size_llama8b_mlp_properties(group):
    """BASELINE config 2 on one rank: 32768 tokens x 4096, w1/w3 [4096,1792], w2 [1792,4096]."""
    torch.manual_seed(0)
    A = torch.randn(32768, 4096, device="cuda").bfloat16()
    w1 = (torch.randn(4096, 1792, device="cuda") * 0.02).bfloat16()
    w3 = (torch.randn(4096, 1792, device="cuda") * 0.02).bfloat16()
    _, (h1, h3) = torch.ops._ap_symm_mem.fused_all_gather_matmul(A, [w1, w3], 0, group, return_A=False)
    _freivalds(h1, A, w1, BF16_TOL)
    _freivalds(h3, A, w3, BF16_TOL)
    # column sums: 1^T C == (1^T A) B
    col_ref = A.double().sum(0) @ w1.double()
    assert ((h1.double().sum(0) - col_ref).norm() / col_ref.norm()).item() <= BF16_TOL
    h = torch.nn.functional.silu(h1.float()).mul_(h3.float()).bfloat16()
    w2 = (torch.randn(1792, 4096, device="cuda") * 0.02).bfloat16()
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(h, w2, "sum", 0, group)
    assert out.shape == (32768, 4096)
    _freivalds(out, h, w2, BF16_TOL)
    # idempotence: the same call gives the same bits
    out2 = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(h, w2, "sum", 0, group)
    assert torch.equal(out, out2)


def test_full_size_llama70b_fp8_properties(group):
    """BASELINE config 4 on one rank: 16384 tokens x 8192 e4m3 row-wise, w1 [8192,3584]."""
    orc = _orc()
    torch.manual_seed(1)
    x = torch.randn(16384, 8192, device="cuda")
    w = torch.randn(8192, 3584, device="cuda") * 0.02
    sa = x.abs().amax(1, keepdim=True) / 448
    sb = w.abs().amax(0, keepdim=True) / 448
    a8 = (x / sa).to(orc.FP8)
    b8 = (w / sb).to(orc.FP8).t().contiguous().t()
    _, (o,) = torch.ops._ap_symm_mem.fused_all_gather_scaled_matmul(
        a8, [b8], sa, [sb], 0, group, [None], [None], [torch.bfloat16], [False]
    )
    g = torch.Generator(device="cuda").manual_seed(5)
    v = torch.randn(3584, 4, device="cuda", dtype=torch.float64, generator=g)
    lhs = o.double() @ v
    rhs = (a8.double() * sa.double()) @ ((b8.double() * sb.double()) @ v)
    assert ((lhs - rhs).norm() / rhs.norm()).item() <= FP8_TOL


def test_full_size_llama8b_attention_properties(group):
    """BASELINE config 3 on one rank: 32768 tokens x 4096, wq/wk/wv [4096, 512 / 128 / 128], wo [512, 4096]
    (mixed output widths in one launch, and a reduce-scatter matmul with only eight k-blocks per tile)."""
    torch.manual_seed(2)
    A = torch.randn(32768, 4096, device="cuda").bfloat16()
    ws = [(torch.randn(4096, n, device="cuda") * 0.02).bfloat16() for n in (512, 128, 128)]
    _, outs = torch.ops._ap_symm_mem.fused_all_gather_matmul(A, ws, 0, group, return_A=False)
    for o, w in zip(outs, ws):
        assert o.shape == (32768, w.shape[1])
        _freivalds(o, A, w, BF16_TOL)
    x = torch.randn(32768, 512, device="cuda").bfloat16()
    wo = (torch.randn(512, 4096, device="cuda") * 0.02).bfloat16()
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(x, wo, "sum", 0, group)
    assert out.shape == (32768, 4096)
    _freivalds(out, x, wo, BF16_TOL)
    avg = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(x, wo, "avg", 0, group)
    assert torch.equal(avg, out)          # a group of one: the mean of one partial is that partial


def test_full_size_llama70b_fp8_reduce_scatter_properties(group):
    """The reduce-scatter side of BASELINE config 4 on one rank: [16384, 3584] e4m3 row-wise x w2 [3584, 8192]
    column-wise -> bf16."""
    orc = _orc()
    torch.manual_seed(3)
    x = torch.randn(16384, 3584, device="cuda")
    w = torch.randn(3584, 8192, device="cuda") * 0.02
    sa = x.abs().amax(1, keepdim=True) / 448
    sb = w.abs().amax(0, keepdim=True) / 448
    a8 = (x / sa).to(orc.FP8)
    b8 = (w / sb).to(orc.FP8).t().contiguous().t()
    out = torch.ops._ap_symm_mem.fused_scaled_matmul_reduce_scatter(
        a8, b8, sa, sb, "sum", 0, 0, group, [16384, 8192], None, None, torch.bfloat16, False
    )
    assert out.shape == (16384, 8192) and out.dtype == torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(5)
    v = torch.randn(8192, 4, device="cuda", dtype=torch.float64, generator=g)
    lhs = out.double() @ v
    rhs = (a8.double() * sa.double()) @ ((b8.double() * sb.double()) @ v)
    assert ((lhs - rhs).norm() / rhs.norm()).item() <= FP8_TOL
    # against the library's own row-wise _scaled_mm on the same operands: both round an fp32 result to bf16
    lib = torch._scaled_mm(a8, b8, sa, sb, out_dtype=torch.bfloat16)
    assert ((out.double() - lib.double()).norm() / lib.double().norm()).item() <= 2 ** -8


def test_scaled_reduce_scatter_with_a_folded_scatter_dim(group):
    """A scatter dim that a pre-matmul reshape folded into the rows (orig_scatter_dim 1, 0 after the reshape,
    output_shape [B, S, N] with B > 1; autoparallel/asynctp.py:896-940 emits it). The reference's CUDA body
    returns row chunk `rank` of the flattened [B*S, N] product viewed as [B, S/world, N]
    (autoparallel/asynctp_ops.py:1375-1423); this is that layout, here on a group of one."""
    orc = _orc()
    Bt, S, K, N = 3, 64, 256, 136
    a8, sa, b8, sb = _fp8_case(orc, Bt * S, K, N, seed=9)
    out = torch.ops._ap_symm_mem.fused_scaled_matmul_reduce_scatter(
        a8.cuda(), b8.cuda().t().contiguous().t(), sa.cuda(), sb.cuda(), "sum", 1, 0, group, [Bt, S, N], None, None,
        torch.bfloat16, False,
    )
    assert out.shape == (Bt, S, N)
    ref64 = ((a8.double() * sa.double()) @ (b8.double() * sb.double())).view(Bt, S, N)     # rows in (b, s) order
    assert orc.rel_fro_error(out, ref64) <= FP8_TOL
    # row r of the flattened product lands at [r // S, r % S]: a probe that differs per row
    row_norm = out.float().flatten(0, 1).norm(dim=1).cpu()
    assert torch.allclose(row_norm, ref64.flatten(0, 1).norm(dim=1).float(), rtol=2e-2)


def test_more_than_four_operands(group):
    """Six Bs share one gathered A: one fused launch for four, one local launch for the rest."""
    from autoparallel_b200 import _native as nat

    orc = _orc()
    A = orc.activations(0, 300, 264)
    Bs = [orc.weights(20 + i, 264, 8 * (i + 3)) for i in range(6)]
    before = nat.lib().apk_launch_count()
    A_out, outs = _ag(A, Bs, 0, group)
    assert nat.lib().apk_launch_count() == before + 2
    assert torch.equal(A_out.cpu(), A)
    for o, b in zip(outs, Bs):
        assert orc.rel_fro_error(o, A.double() @ b.double()) <= BF16_TOL


@pytest.mark.parametrize("b_layout", ["row_major", "transposed_view"])
def test_float16_operands(group, b_layout):
    """float16 A and B (the reference forwards any dtype to aten.mm, autoparallel/asynctp_ops.py:519, :1168):
    same kernels, IEEE-half operand format and outputs. Tolerance as for bf16; half has three more mantissa bits."""
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randn(1000, 1032, device="cuda", generator=g).half()
    Bs = [(torch.randn(1032, n, device="cuda", generator=g) * 0.05).half() for n in (264, 512)]
    if b_layout == "transposed_view":
        Bs = [b.t().contiguous().t() for b in Bs]
    A_out, outs = torch.ops._ap_symm_mem.fused_all_gather_matmul(A, Bs, 0, group)
    assert torch.equal(A_out, A)
    for o, b in zip(outs, Bs):
        assert o.dtype == torch.float16
        e = ((o.double() - A.double() @ b.double()).norm() / (A.double() @ b.double()).norm()).item()
        assert e <= BF16_TOL / 4, e
        lib = A @ b                       # cuBLAS, fp32 accumulate, rounded to half
        assert ((o.double() - lib.double()).norm() / lib.double().norm()).item() <= 2 ** -10
    w2 = (torch.randn(264, 520, device="cuda", generator=g) * 0.05).half()
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(outs[0], w2, "avg", 0, group)
    ref = outs[0].double() @ w2.double()
    assert out.dtype == torch.float16 and ((out.double() - ref).norm() / ref.norm()).item() <= BF16_TOL / 4


def test_timeline_stamps_are_ordered(group):
    """apk_set_trace: every tile of a launch leaves one record, and inside a record the stamps follow the
    pipeline: first load <= first MMA <= last MMA committed <= accumulator complete <= epilogue done, all
    inside the CTA's own begin / end."""
    from autoparallel_b200 import timeline

    A = torch.randn(4096, 1024, device="cuda").bfloat16()
    B = (torch.randn(1024, 512, device="cuda") * 0.02).bfloat16()
    dev = torch.device("cuda", 0)
    with timeline.capture(dev) as tl:
        torch.ops._ap_symm_mem.fused_all_gather_matmul(A, [B], 0, group, return_A=False)
        rec = tl.records()
    F = timeline.F
    used = rec[rec[:, F["tile"]] > 0]
    tiles = (4096 // 128) * (512 // 256)
    assert used.shape[0] == tiles and sorted((used[:, F["tile"]] - 1).tolist()) == sorted(list(range(tiles // 2)) * 2)   # pairs: both CTAs record
    mma = used[used[:, F["mma_t"]] > 0]          # the CTA of a pair that issues the MMAs
    assert mma.shape[0] == tiles // 2
    assert bool((mma[:, F["load_t"]] <= mma[:, F["mma_t"]]).all())
    assert bool((mma[:, F["mma_t"]] <= mma[:, F["commit_t"]]).all())
    assert bool((mma[:, F["commit_t"]] <= mma[:, F["tfull_t"]] + 1000).all())   # globaltimer ticks are coarse (up to 1 us)
    assert bool((used[:, F["tfull_t"]] <= used[:, F["epi_end_t"]]).all())
    s = timeline.summary(rec)
    assert s["tiles"] == tiles and 0 < s["span_us"] < 1e4 and 500 < s["sm_mhz_in_kernel"] < 2500
    # off again: a launch after the capture leaves the (zeroed) buffer alone
    tl.clear()
    torch.ops._ap_symm_mem.fused_all_gather_matmul(A, [B], 0, group, return_A=False)
    torch.cuda.synchronize()
    assert int(tl.buf.abs().sum()) == 0


# --------------------------------------------------------------------------------------- C ABI, status word
def test_c_abi_direct_call_and_alignment_error(group):
    from autoparallel_b200 import _native as nat

    L = nat.lib()
    orc = _orc()
    A = orc.activations(0, 256, 128).cuda()
    B = orc.weights(7, 128, 64).cuda()
    out = torch.empty(256, 64, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    comm = nat.ApkComm()
    comm.rank, comm.world, comm.status, comm.epoch, comm.timeout_s = 0, 1, status.data_ptr(), 1, 5.0
    args = nat.ApkAgGemmArgs()
    args.dtype, args.rows_per_rank, args.K, args.nB = nat.APK_BF16, 256, 128, 1
    args.A_shard, args.lda = A.data_ptr(), 128
    op = args.Bs[0]
    op.B, op.ldb, op.n_major, op.N = B.data_ptr(), 64, 1, 64
    op.out, op.ldo, op.out_dtype = out.data_ptr(), 64, nat.APK_BF16
    before = L.apk_launch_count()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.apk_ag_gemm(C.byref(comm), C.byref(args), stream) == nat.APK_OK
    assert L.apk_launch_count() == before + 1
    raw = C.c_uint32(7)
    assert L.apk_check_status(C.byref(comm), stream, C.byref(raw)) == nat.APK_OK and raw.value == 0
    assert orc.rel_fro_error(out, A.double().cpu() @ B.double().cpu()) <= BF16_TOL
    args.A_shard = A.data_ptr() + 2  # not 16-byte aligned: rejected before any launch
    assert L.apk_ag_gemm(C.byref(comm), C.byref(args), stream) == nat.APK_ERR_ARG
    assert b"16-byte aligned" in L.apk_last_error()


def _to_blocked(part, BN):
    """[rows, N] bf16 partial -> the arena's layout for one source rank: per 128 x BN tile (row block
    major), per 64-column group, per 32-row quarter, a contiguous [32, 64] block."""
    rows, N = part.shape
    mt, nt = (rows + 127) // 128, (N + BN - 1) // BN
    pad = torch.zeros(mt * 128, nt * BN, dtype=part.dtype, device=part.device)
    pad[:rows, :N] = part
    blocks = pad.view(mt, 4, 32, nt, BN // 64, 64).permute(0, 3, 4, 1, 2, 5).contiguous().view(-1, 32, 8, 8)
    pos = torch.arange(8, device=part.device)[None, :] ^ (torch.arange(32, device=part.device) % 8)[:, None]
    idx = pos[None, :, :, None].expand(blocks.shape[0], 32, 8, 8)
    return blocks.gather(2, idx).contiguous().view(-1)


@pytest.mark.parametrize("world,M,K,N", [(2, 512, 256, 256), (4, 4 * 384, 192, 328), (8, 8 * 128, 128, 64)])
def test_reduce_scatter_receive_side_on_one_gpu(group, world, M, K, N):
    """Rank 0 of a `world`-rank reduce-scatter on a single GPU: the peers' partials for rank 0's rows
    are placed in its arena beforehand and their tile flags are set, so the epilogue's wait, its
    read of the blocked arena and the fp32 sum run exactly as with live peers. What rank 0 sends
    to the others lands in scratch arenas and is checked too."""
    from autoparallel_b200 import _native as nat

    L = nat.lib()
    orc = _orc()
    rows = M // world
    BN = 128 if N <= 128 else 256
    A = orc.activations(0, M, K)
    B = orc.weights(7, K, N)
    peers = [orc.activations(10 + r, rows, N) * 0.3 for r in range(world)]   # bf16 partials of ranks 1..world-1
    args0 = nat.ApkGemmRsArgs()
    args0.M, args0.B.N, args0.B.out_dtype = M, N, nat.APK_BF16
    half = int(L.apk_gemm_rs_arena_bytes(C.byref(args0), world))
    slot = half // (world + 2)   # world source slots, then the fp32 sums (two slots' worth)
    arenas = [torch.zeros(2 * half, dtype=torch.uint8, device="cuda") for _ in range(world)]
    for h in range(2):
        for src in range(1, world):
            blk = _to_blocked(peers[src].cuda(), BN).view(torch.uint8)
            arenas[0][h * half + src * slot: h * half + src * slot + blk.numel()] = blk
    pads = [torch.zeros(1 << 17, dtype=torch.int32, device="cuda") for _ in range(world)]
    pads[0][1024:] = 1000      # every (source, tile) flag of rank 0 is already raised (tile flags start at byte 4096)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctrl = torch.zeros(1024, dtype=torch.int32, device="cuda")
    Ad, Bd = A.cuda(), B.cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    full64 = A.double() @ B.double()
    for epoch in (1, 2):
        out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        comm = nat.ApkComm()
        comm.rank, comm.world = 0, world
        for r in range(world):
            comm.data[r], comm.flags[r] = arenas[r].data_ptr(), pads[r].data_ptr()
        comm.data_bytes, comm.flag_bytes = 2 * half, pads[0].numel() * 4
        comm.ctrl, comm.ctrl_bytes = ctrl.data_ptr(), ctrl.numel() * 4
        comm.status, comm.epoch, comm.timeout_s = status.data_ptr(), epoch, 5.0
        args = nat.ApkGemmRsArgs()
        args.dtype, args.M, args.K, args.reduce_op = nat.APK_BF16, M, K, nat.APK_REDUCE_AVG
        args.A, args.lda = Ad.data_ptr(), K
        args.B.B, args.B.ldb, args.B.n_major, args.B.N = Bd.data_ptr(), N, 1, N
        args.B.out, args.B.ldo, args.B.out_dtype = out.data_ptr(), N, nat.APK_BF16
        assert L.apk_gemm_rs(C.byref(comm), C.byref(args), stream) == nat.APK_OK, L.apk_last_error()
        raw = C.c_uint32(0)
        assert L.apk_check_status(C.byref(comm), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()
        ref64 = (full64[:rows] + sum(peers[s].double() for s in range(1, world))) / world
        assert orc.rel_fro_error(out, ref64) <= BF16_TOL
        # what went out: peer d's arena, slot 0, holds rows [d*rows, (d+1)*rows) of A @ B in blocked form
        off = (epoch & 1) * half
        for d in range(1, world):
            want = _to_blocked(full64[d * rows:(d + 1) * rows].to(torch.bfloat16).cuda(), BN)
            got = arenas[d][off: off + want.numel() * 2].view(torch.bfloat16)
            mask = want != 0   # padding columns / rows of a block are not specified
            assert orc.rel_fro_error(got[mask].float(), want[mask].double().cpu()) <= BF16_TOL
            assert int(pads[d][1024 + 0]) == epoch   # flag (source 0, tile 0) released with the epoch


def test_reduce_scatter_fp32_partials_receive_side_on_one_gpu(group):
    """fp32 outputs travel as fp32 partials in row-major slots (the bf16 path uses the blocked arena):
    rank 1 of a three-rank group on one GPU, peers' partials and flags placed beforehand."""
    from autoparallel_b200 import _native as nat

    L = nat.lib()
    orc = _orc()
    world, rank, M, K, N = 3, 1, 3 * 200, 128, 72
    rows, slot_rows = M // world, 256
    A, B = orc.activations(0, M, K), orc.weights(7, K, N)
    peers = {r: torch.randn(rows, N) for r in (0, 2)}
    args0 = nat.ApkGemmRsArgs()
    args0.M, args0.B.N, args0.B.out_dtype = M, N, nat.APK_F32
    half = int(L.apk_gemm_rs_arena_bytes(C.byref(args0), world))
    assert half == world * slot_rows * N * 4
    arenas = [torch.zeros(2 * half, dtype=torch.uint8, device="cuda") for _ in range(world)]
    for h in range(2):
        for src, part in peers.items():
            off = h * half + src * slot_rows * N * 4
            arenas[rank][off: off + rows * N * 4] = part.cuda().view(torch.uint8).view(-1)
    pads = [torch.zeros(1 << 17, dtype=torch.int32, device="cuda") for _ in range(world)]
    pads[rank][1024:] = 1000
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctrl = torch.zeros(1024, dtype=torch.int32, device="cuda")
    Ad, Bd = A.cuda(), B.cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    full64 = A.double() @ B.double()
    for epoch in (1, 2):
        out = torch.full((rows, N), float("nan"), dtype=torch.float32, device="cuda")
        comm = nat.ApkComm()
        comm.rank, comm.world = rank, world
        for r in range(world):
            comm.data[r], comm.flags[r] = arenas[r].data_ptr(), pads[r].data_ptr()
        comm.data_bytes, comm.flag_bytes = 2 * half, pads[0].numel() * 4
        comm.ctrl, comm.ctrl_bytes = ctrl.data_ptr(), ctrl.numel() * 4
        comm.status, comm.epoch, comm.timeout_s = status.data_ptr(), epoch, 5.0
        args = nat.ApkGemmRsArgs()
        args.dtype, args.M, args.K, args.reduce_op = nat.APK_BF16, M, K, nat.APK_REDUCE_SUM
        args.A, args.lda = Ad.data_ptr(), K
        args.B.B, args.B.ldb, args.B.n_major, args.B.N = Bd.data_ptr(), N, 1, N
        args.B.out, args.B.ldo, args.B.out_dtype = out.data_ptr(), N, nat.APK_F32
        assert L.apk_gemm_rs(C.byref(comm), C.byref(args), stream) == nat.APK_OK, L.apk_last_error()
        raw = C.c_uint32(0)
        assert L.apk_check_status(C.byref(comm), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()
        ref64 = full64[rank * rows:(rank + 1) * rows] + sum(p.double() for p in peers.values())
        assert orc.rel_fro_error(out, ref64) <= 1e-5
        # the part sent to rank 2: slot `rank` of its arena, fp32 row-major
        off = (epoch & 1) * half + rank * slot_rows * N * 4
        sent = arenas[2][off: off + rows * N * 4].view(torch.float32).view(rows, N)
        assert orc.rel_fro_error(sent, full64[2 * rows:]) <= 1e-5


def test_device_wait_times_out_cleanly(group):
    """A two-rank reduce-scatter whose 'peer' is this GPU's own memory and never answers: the
    wait for the peer's partial runs out after timeout_s, the kernel frees its resources and
    returns, the status word says which wait gave up, and the context stays usable."""
    from autoparallel_b200 import _native as nat

    L = nat.lib()
    orc = _orc()
    M, K, N = 256, 64, 64
    A = orc.activations(0, M, K).cuda()
    B = orc.weights(7, K, N).cuda()
    out = torch.empty(M // 2, N, dtype=torch.bfloat16, device="cuda")
    arena = torch.zeros(2 * 4 * 128 * 128, dtype=torch.bfloat16, device="cuda")  # two halves of [2 rank slots + fp32 sums][1 tile of 128x128]
    flags = torch.zeros(8192 * 2, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctrl = torch.zeros(1024, dtype=torch.int32, device="cuda")
    comm = nat.ApkComm()
    comm.rank, comm.world = 0, 2
    for r in range(2):
        comm.data[r] = arena.data_ptr()
        comm.flags[r] = flags.data_ptr()
    comm.data_bytes, comm.flag_bytes = arena.numel() * 2, flags.numel() * 4
    comm.ctrl, comm.ctrl_bytes = ctrl.data_ptr(), ctrl.numel() * 4
    comm.status, comm.epoch, comm.timeout_s = status.data_ptr(), 1, 0.2
    args = nat.ApkGemmRsArgs()
    args.dtype, args.M, args.K, args.reduce_op = nat.APK_BF16, M, K, nat.APK_REDUCE_SUM
    args.A, args.lda = A.data_ptr(), K
    args.B.B, args.B.ldb, args.B.n_major, args.B.N = B.data_ptr(), N, 1, N
    args.B.out, args.B.ldo, args.B.out_dtype = out.data_ptr(), N, nat.APK_BF16
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.apk_gemm_rs(C.byref(comm), C.byref(args), stream) == nat.APK_OK
    raw = C.c_uint32(0)
    assert L.apk_check_status(C.byref(comm), stream, C.byref(raw)) == nat.APK_ERR_TIMEOUT
    assert raw.value & 0xFF == 4 and raw.value >> 8 == 1  # peer partial, source rank 1
    assert b"peer partial" in L.apk_last_error()
    # the partial for the other rank was still produced, and the device still works
    # (epoch 1 uses the second half of the arena; its first tile holds what rank 0 sent, in the
    #  arena's blocked layout)
    half = arena.numel() // 2
    want = _to_blocked((A.double().cpu() @ B.double().cpu())[M // 2:].to(torch.bfloat16).cuda(), 128)
    got = arena[half: half + want.numel()]
    mask = want != 0
    assert orc.rel_fro_error(got[mask].float(), want[mask].double().cpu()) <= BF16_TOL
    assert L.apk_check_status(C.byref(comm), stream, C.byref(raw)) == nat.APK_OK
    assert float((A.float() @ B.float()).sum()) == float((A.float() @ B.float()).sum())
