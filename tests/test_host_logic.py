"""Host-side mirror of autoparallel/asynctp_ops.py: schemas, helpers, Meta kernels, error
behaviour, and the drop-in installation under the reference's unchanged FX pass."""
import os
import sys

import pytest
import torch
import torch.distributed as dist

import autoparallel_b200.asynctp_ops as ops
from autoparallel_b200.install import install

# The AutoParallel source tree: $AUTOPARALLEL_REFERENCE, or a checkout named `reference` beside this repository.
REFERENCE = os.environ.get("AUTOPARALLEL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


@pytest.fixture(scope="module")
def fake_pg():
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=8)
    yield dist.group.WORLD.group_name
    dist.destroy_process_group()


def test_schemas_match_reference_text():
    ns = torch.ops._ap_symm_mem
    assert str(ns.fused_all_gather_matmul.default._schema) == (
        "_ap_symm_mem::fused_all_gather_matmul(Tensor A, Tensor[] Bs, int gather_dim, str group_name, *, "
        "bool return_A=True) -> (Tensor?, Tensor[])"
    )
    assert str(ns.fused_matmul_reduce_scatter.default._schema) == (
        "_ap_symm_mem::fused_matmul_reduce_scatter(Tensor A, Tensor B, str reduce_op, int scatter_dim, "
        "str group_name) -> Tensor"
    )
    assert "ScalarType?[] out_dtypes, bool[] use_fast_accum) -> (Tensor, Tensor[])" in str(
        ns.fused_all_gather_scaled_matmul.default._schema
    )
    assert "int[]? output_shape, Tensor? bias=None, Tensor? result_scale=None, ScalarType? out_dtype=None, bool use_fast_accum=False) -> Tensor" in str(
        ns.fused_scaled_matmul_reduce_scatter.default._schema
    )
    for name in ("fused_all_gather_matmul", "fused_all_gather_scaled_matmul", "fused_matmul_reduce_scatter",
                 "fused_scaled_matmul_reduce_scatter"):
        assert torch._C.Tag.needs_fixed_stride_order in getattr(ns, name).default.tags
    assert hasattr(ns, "_low_contention_all_gather") and hasattr(ns, "_low_contention_reduce_scatter")


def test_scale_mode_classifier():
    M = ops._ScaleMode
    f = ops._check_and_verify_fp8_all_gather_scale_mode
    shard = torch.empty(4, 6, 8)
    assert f(shard, None, 0, 2) is M.UNSCALED
    assert f(shard, torch.empty(4, 6, 1), 0, 2) is M.ROW_WISE_SHARDED
    assert f(shard, torch.tensor(1.0), 0, 2) is M.TENSOR_WISE
    assert f(shard, torch.empty(1, 1), 0, 2) is M.TENSOR_WISE
    assert f(shard, torch.empty(8, 6, 1), 0, 2) is M.ROW_WISE_REPLICATED
    assert f(shard, torch.empty(4, 12, 1), 1, 2) is M.ROW_WISE_REPLICATED
    # ambiguous [.., 1] shard is treated as row-wise sharded, like the reference
    assert f(torch.empty(1, 1), torch.empty(1, 1), 0, 2) is M.ROW_WISE_SHARDED
    with pytest.raises(ValueError, match="Invalid scale shape"):
        f(shard, torch.empty(3, 6, 1), 0, 2)


def test_scalar_type_conversion():
    f = ops._maybe_convert_scalar_types_to_dtypes
    assert f([15, None, 6, 17]) == [torch.bfloat16, None, torch.float32, torch.float8_e4m3fn]
    assert f([torch.bfloat16, None]) == [torch.bfloat16, None]
    with pytest.raises(ValueError):
        f([99])


def test_restride_helpers():
    t = torch.arange(2 * 3 * 4).view(2, 3, 4)
    r = ops.restride_A_shard_for_fused_all_gather_matmul(t, 1)
    assert torch.equal(r, t) and r.movedim(1, 0).is_contiguous()
    r = ops.restride_A_for_fused_matmul_reduce_scatter(t, 2)
    assert torch.equal(r, t) and r.movedim(2, 0).is_contiguous()
    p = ops.make_contiguous_for_perm(t, [2, 0, 1])
    assert torch.equal(p, t) and p.permute(2, 0, 1).is_contiguous()


def test_meta_shapes(fake_pg):
    g = fake_pg
    A = torch.empty(4, 6, 64, device="meta", dtype=torch.bfloat16)
    Bs = [torch.empty(64, 40, device="meta", dtype=torch.bfloat16), torch.empty(64, 24, device="meta", dtype=torch.bfloat16)]
    for gd, shape in ((0, (32, 6)), (1, (4, 48))):
        Aout, outs = torch.ops._ap_symm_mem.fused_all_gather_matmul(A, Bs, gd, g)
        assert tuple(Aout.shape) == (*shape, 64)
        assert [tuple(o.shape) for o in outs] == [(*shape, 40), (*shape, 24)]
        Aout, _ = torch.ops._ap_symm_mem.fused_all_gather_matmul(A, Bs, gd, g, return_A=False)
        assert Aout is None
    X = torch.empty(16, 6, 64, device="meta", dtype=torch.bfloat16)
    out = torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(X, Bs[0], "sum", 0, g)
    assert tuple(out.shape) == (2, 6, 40) and out.dtype == torch.bfloat16


def test_cpu_tensors_have_no_kernel(fake_pg):
    """There is no CPU path: the ops exist for Meta and CUDA only, as in the reference."""
    with pytest.raises(NotImplementedError):
        torch.ops._ap_symm_mem.fused_matmul_reduce_scatter(torch.zeros(8, 8), torch.zeros(8, 8), "sum", 0, fake_pg)


def test_argument_errors_match_reference(fake_pg):
    g = fake_pg
    bf = torch.bfloat16
    A, B = torch.empty(8, 64, dtype=bf), torch.empty(64, 16, dtype=bf)
    n = [None]
    with pytest.raises(ValueError, match="A_shard must be a matrix"):
        ops._ag_gemm_native(torch.empty(8, dtype=bf), [B], None, n, n, n, [bf], 0, g, True)
    with pytest.raises(ValueError, match="B must be a matrix"):
        ops._ag_gemm_native(A, [torch.empty(64, dtype=bf)], None, n, n, n, [bf], 0, g, True)
    with pytest.raises(ValueError, match="Invalid gather_dim"):
        ops._ag_gemm_native(A, [B], None, n, n, n, [bf], 2, g, True)
    with pytest.raises(ValueError, match="len\\(out_types\\)"):
        ops._ag_gemm_native(A, [B], None, n, n, n, [], 0, g, True)
    with pytest.raises(ValueError, match="gathered A has 512 columns"):   # last-dim gather: B must span all K-slices
        ops._ag_gemm_native(A, [B], None, n, n, n, [bf], 1, g, True)
    with pytest.raises(NotImplementedError, match="bfloat16, float16 or float8_e4m3fn"):
        ops._ag_gemm_native(A.float(), [B.float()], None, n, n, n, [torch.float32], 0, g, True)
    with pytest.raises(ValueError, match="reduce_op must be sum or avg"):
        ops._check_reduce_op("max")
    with pytest.raises(ValueError, match="len\\(biases\\)"):
        ops._fused_all_gather_scaled_matmul(A, [B], torch.tensor(1.0), [torch.tensor(1.0)], 0, g, [], [None], [bf], [False])


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="AutoParallel sources not present")
def test_unchanged_fx_pass_targets_the_drop_in(fake_pg):
    """The reference's micro_pipeline_tp_pass, imported unmodified, rewrites AG->mm,mm->silu*mul->mm->RS
    into this package's fused ops."""
    import torch.distributed._functional_collectives as funcol
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.distributed._symmetric_memory import _test_mode
    from torch.fx.experimental.proxy_tensor import make_fx

    install()
    sys.path.insert(0, REFERENCE)
    try:
        import autoparallel.asynctp as asynctp
    finally:
        sys.path.remove(REFERENCE)
    assert sys.modules["autoparallel.asynctp_ops"] is ops
    g = fake_pg

    def mlp(x, w1, w3, w2):
        a = funcol.all_gather_tensor(x, 0, g)
        h = torch.nn.functional.silu(a @ w1) * (a @ w3)
        return funcol.reduce_scatter_tensor(h @ w2, "sum", 0, g)

    with FakeTensorMode():
        bf = torch.bfloat16
        x = torch.empty(512, 4096, dtype=bf, device="cuda")
        w1 = torch.empty(4096, 1792, dtype=bf, device="cuda")
        w3 = torch.empty(4096, 1792, dtype=bf, device="cuda")
        w2 = torch.empty(1792, 4096, dtype=bf, device="cuda")
        gm = make_fx(mlp, tracing_mode="fake")(x, w1, w3, w2)
    with _test_mode():
        asynctp.micro_pipeline_tp_pass(gm.graph)
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert torch.ops._ap_symm_mem.fused_all_gather_matmul.default in targets
    assert torch.ops._ap_symm_mem.fused_matmul_reduce_scatter.default in targets
    assert torch.ops._c10d_functional.all_gather_into_tensor.default not in targets
    assert torch.ops._c10d_functional.reduce_scatter_tensor.default not in targets
    ag = next(n for n in gm.graph.nodes if n.target == torch.ops._ap_symm_mem.fused_all_gather_matmul.default)
    assert len(ag.args[1]) == 2 and ag.kwargs.get("return_A") is False


def test_torch_pass_can_be_retargeted_to_these_ops(fake_pg):
    """torch's own micro-pipeline pass (which AutoParallel's is a fork of) inserts the same calls under
    torch.ops.symm_mem; install.retarget_symm_mem_calls points them at this package's ops, arguments untouched.
    (This is what tests/test_gpu_compiled_graph.py runs under torch.compile on GPUs.)"""
    import torch.distributed._functional_collectives as funcol
    from torch._inductor.fx_passes.micro_pipeline_tp import micro_pipeline_tp_pass
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.distributed._symmetric_memory import _test_mode
    from torch.fx.experimental.proxy_tensor import make_fx

    from autoparallel_b200.install import retarget_symm_mem_calls

    g = fake_pg

    def f(x, w1, w3, w2):
        a = funcol.all_gather_tensor(x, 0, g)
        h = torch.nn.functional.silu(a @ w1) * (a @ w3)
        return funcol.reduce_scatter_tensor(h @ w2, "sum", 0, g)

    with FakeTensorMode():
        args = [torch.empty(s, dtype=torch.bfloat16, device="cuda") for s in ((512, 1024), (1024, 256), (1024, 256), (256, 1024))]
        gm = make_fx(f, tracing_mode="fake")(*args)
    with _test_mode():
        micro_pipeline_tp_pass(gm.graph)
    before = [str(n.args) for n in gm.graph.nodes if n.op == "call_function" and "symm_mem.fused" in str(n.target)]
    assert retarget_symm_mem_calls(gm.graph) == 2
    gm.graph.lint()
    ns = torch.ops._ap_symm_mem
    after = {n.target: str(n.args) for n in gm.graph.nodes if n.op == "call_function" and "_ap_symm_mem" in str(n.target)}
    assert set(after) == {ns.fused_all_gather_matmul.default, ns.fused_matmul_reduce_scatter.default}
    assert sorted(before) == sorted(after.values())              # same arguments
    assert retarget_symm_mem_calls(gm.graph) == 0                 # idempotent
