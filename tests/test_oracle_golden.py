"""The CPU oracle against outputs of the reference's own fallbacks (tests/golden/asynctp_golden.pt,
made by tests/golden/make_golden.py from autoparallel/asynctp_ops.py:672-700, :1090-1100, :1242-1290)."""
import pytest
import torch

from oracle import asynctp_oracle as orc


def _cases(golden, kind):
    r0, r1 = golden["ranks"]
    return [(a, b) for a, b in zip(r0, r1) if a["kind"] == kind]


def test_fixture_is_complete(golden):
    kinds = [c["kind"] for c in golden["ranks"][0]]
    assert golden["world"] == 2
    assert kinds.count("ag_mm") == 8 and kinds.count("mm_rs") == 12 and kinds.count("smm_rs") == 2
    assert kinds.count("config1") == 1


def test_all_gather_matmul_matches_reference(golden):
    for c0, c1 in _cases(golden, "ag_mm"):
        A, outs = orc.all_gather_matmul_local([c0["A_shard"], c1["A_shard"]], c0["Bs"], c0["gather_dim"], return_A=True)
        for rec in (c0, c1):  # every rank holds the same gathered result
            assert A.shape == rec["A_out"].shape and A.dtype == rec["A_out"].dtype
            assert torch.equal(A, rec["A_out"]), (c0["shape"], c0["gather_dim"])
            for o, g in zip(outs, rec["outs"]):
                assert o.shape == g.shape and o.dtype == g.dtype
                torch.testing.assert_close(o, g, rtol=0, atol=0)


def test_all_gather_matmul_return_A_false(golden):
    c0, c1 = _cases(golden, "ag_mm")[0]
    A, outs = orc.all_gather_matmul_local([c0["A_shard"], c1["A_shard"]], c0["Bs"], 0, return_A=False)
    assert A is None and len(outs) == 2


def test_matmul_reduce_scatter_matches_reference(golden):
    for c0, c1 in _cases(golden, "mm_rs"):
        outs = orc.matmul_reduce_scatter_local([c0["A"], c1["A"]], [c0["B"], c1["B"]], c0["op"], c0["scatter_dim"])
        for o, rec in zip(outs, (c0, c1)):
            assert o.shape == rec["out"].shape and o.dtype == rec["out"].dtype
            if o.dtype == torch.float32:
                torch.testing.assert_close(o, rec["out"], rtol=1e-6, atol=1e-6)
            else:
                # gloo adds bf16 partials in bf16; the oracle adds in fp32 and rounds once:
                # at most one bf16 ulp apart.
                torch.testing.assert_close(o.float(), rec["out"].float(), rtol=2 ** -7, atol=1e-3)


def test_scaled_matmul_reduce_scatter_matches_reference(golden):
    for c0, c1 in _cases(golden, "smm_rs"):
        Bs = [c0["B_t"].t(), c1["B_t"].t()]
        outs = orc.scaled_matmul_reduce_scatter_local(
            [c0["A"], c1["A"]], Bs, [c0["A_scale"], c1["A_scale"]], [c0["B_scale"], c1["B_scale"]],
            c0["op"], 0, [c0["shape"][0], c0["N"]], out_dtype=torch.bfloat16,
        )
        for o, rec in zip(outs, (c0, c1)):
            assert o.shape == rec["out"].shape and o.dtype == rec["out"].dtype
            torch.testing.assert_close(o.float(), rec["out"].float(), rtol=2 ** -7, atol=1e-3)


def test_config1_digest(golden):
    """BASELINE config 1 at full size: fp32 A_shard [512,1024] per rank, B [1024,2048], W2 [2048,1024]."""
    (c0, c1), = _cases(golden, "config1")

    def rnd(seed, *shape, std=1.0):
        g = torch.Generator().manual_seed(seed)
        return torch.randn(*shape, generator=g) * std

    shards = [rnd(1000 + r, 512, 1024) for r in range(2)]
    B, W2 = rnd(7, 1024, 2048, std=0.02), rnd(8, 2048, 1024, std=0.02)
    _, (C1,) = orc.all_gather_matmul_local(shards, [B], 0, return_A=False)
    outs = orc.matmul_reduce_scatter_local([C1, C1], [W2, W2], "sum", 0)
    idx = torch.arange(0, C1.numel(), 509)
    torch.testing.assert_close(C1.flatten()[idx], c0["C_digest"]["sample"], rtol=1e-5, atol=1e-5)
    assert C1.double().sum().item() == pytest.approx(c0["C_digest"]["sum"], rel=1e-6, abs=1e-3)
    for o, rec in zip(outs, (c0, c1)):
        d = rec["out_digest"]
        assert tuple(o.shape) == d["shape"]
        idx = torch.arange(0, o.numel(), 509)
        torch.testing.assert_close(o.flatten()[idx], d["sample"], rtol=1e-5, atol=1e-5)
        assert o.double().abs().sum().item() == pytest.approx(d["abs_sum"], rel=1e-6)


def test_scaled_mm_rowwise_restatement():
    """Row-wise scaling equals dequantise-then-matmul in fp64 up to fp32 rounding."""
    torch.manual_seed(0)
    x, w = torch.randn(32, 64), torch.randn(64, 48) * 0.02
    a8, sa = orc.quantize_rowwise(x, dim=1)
    b8, sb = orc.quantize_rowwise(w, dim=0)
    out = orc.scaled_mm(a8, b8, sa, sb, out_dtype=torch.float32)
    ref = (a8.double() * sa.double()) @ (b8.double() * sb.double())
    assert orc.rel_fro_error(out, ref) < 1e-6
    # and the quantised product is close to the unquantised one
    assert orc.rel_fro_error(out, x.double() @ w.double()) < 6e-2


def test_scaled_all_gather_scale_modes():
    torch.manual_seed(1)
    shards = [torch.randn(8, 16).to(orc.FP8) for _ in range(2)]
    B = (torch.randn(16, 24) * 0.1).to(orc.FP8)
    sb = torch.rand(1, 24) + 0.5
    row = [torch.rand(8, 1) + 0.5 for _ in range(2)]
    full = torch.cat(row)
    A1, (o1,) = orc.all_gather_scaled_matmul_local(shards, [B], row, [sb], 0, [None], [None], [torch.float32])
    A2, (o2,) = orc.all_gather_scaled_matmul_local(shards, [B], [full, full], [sb], 0, [None], [None], [torch.float32])
    assert torch.equal(A1.view(torch.uint8), A2.view(torch.uint8))
    torch.testing.assert_close(o1, o2)
    t = torch.tensor(0.5)
    _, (o3,) = orc.all_gather_scaled_matmul_local(shards, [B], [t, t], [sb], 0, [None], [None], [torch.float32])
    ref = (torch.cat(shards).double() * 0.5) @ (B.double() * sb.double())
    assert orc.rel_fro_error(o3, ref) < 1e-6
    with pytest.raises(ValueError):
        orc.all_gather_scaled_matmul_local(shards, [B], [torch.rand(3, 1)] * 2, [sb], 0, [None], [None], [torch.float32])


# ---- fp8 fixtures made by tests/golden/make_golden_fp8.py (reference fallbacks :873-944 and :1242-1290 over a
# ---- threaded two-rank process group; see that script for what "torch-cpu" and "stand-in" mean)
_DT = {"torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}


def _close_fp8(o, g):
    assert o.shape == g.shape and o.dtype == g.dtype
    if o.dtype == torch.float32:
        torch.testing.assert_close(o, g, rtol=1e-5, atol=1e-5)
    else:  # one bf16 ulp: the two sides may round a differently-ordered fp32 sum
        torch.testing.assert_close(o.float(), g.float(), rtol=2 ** -7, atol=1e-3)


def test_fp8_fixture_is_complete(golden_fp8):
    r0 = golden_fp8["ranks"][0]
    assert golden_fp8["world"] == 2 and len(golden_fp8["ranks"]) == 2
    assert sum(c["kind"] == "sag_mm" and c["scaled_mm"] == "torch-cpu" for c in r0) == 3
    assert sum(c["kind"] == "sag_mm" and c["scaled_mm"] == "stand-in" for c in r0) == 6
    assert sum(c["kind"] == "smm_rs" for c in r0) == 3
    assert {c["mode"] for c in r0} == {"tensor", "row_sharded", "row_replicated", "row"}


def test_all_gather_scaled_matmul_matches_reference(golden_fp8):
    for c0, c1 in _cases(golden_fp8, "sag_mm"):
        Bs = [bt.t() for bt in c0["Bs_t"]]
        A, outs = orc.all_gather_scaled_matmul_local(
            [c0["A_shard"], c1["A_shard"]], Bs, [c0["A_scale"], c1["A_scale"]], c0["B_scales"], c0["gather_dim"],
            c0["biases"], c0["result_scales"], [_DT[d] for d in c0["out_dtypes"]],
        )
        for rec in (c0, c1):
            what = (rec["mode"], rec["shape"], rec["gather_dim"])
            assert A.shape == rec["A_out"].shape and A.dtype == rec["A_out"].dtype, what
            assert torch.equal(A.contiguous().view(torch.uint8), rec["A_out"].view(torch.uint8)), what
            assert len(outs) == len(rec["outs"])
            for o, g in zip(outs, rec["outs"]):
                _close_fp8(o, g)


def test_rowwise_scaled_matmul_reduce_scatter_matches_reference(golden_fp8):
    for c0, c1 in _cases(golden_fp8, "smm_rs"):
        outs = orc.scaled_matmul_reduce_scatter_local(
            [c0["A"], c1["A"]], [c0["B_t"].t(), c1["B_t"].t()], [c0["A_scale"], c1["A_scale"]],
            [c0["B_scale"], c1["B_scale"]], c0["op"], c0["scatter_dim"], c0["output_shape"], out_dtype=torch.bfloat16,
        )
        for o, rec in zip(outs, (c0, c1)):
            _close_fp8(o, rec["out"])
