"""The reference's FX rewrite pass (autoparallel/asynctp.py::micro_pipeline_tp_pass, :1264-1328),
imported unmodified, must emit calls of this package's ops for every pattern it knows: first-dim
and last-dim gather/scatter, the transposed-matmul fusion (off by default, asynctp.py:37) and the
row-wise fp8 ``_scaled_mm`` forms. The graphs are traced on fake tensors over a fake 8-rank
process group, so the tests need neither GPUs nor peers; the arguments of the emitted nodes are
then checked against what the CUDA path accepts (operand layouts are exercised on a GPU in
``test_gpu_single.py``: ``transposed_view`` B, non-contiguous A, fp8 column-major B).
"""
from __future__ import annotations

import operator
import os
import sys

import pytest
import torch
import torch.distributed as dist

import autoparallel_b200.asynctp_ops as ops
from autoparallel_b200.install import install

# The AutoParallel source tree: $AUTOPARALLEL_REFERENCE, or a checkout named `reference` beside this repository.
REFERENCE = os.environ.get("AUTOPARALLEL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="AutoParallel sources not present")

BF, F8, F32 = torch.bfloat16, torch.float8_e4m3fn, torch.float32
NS = torch.ops._ap_symm_mem
C10D = torch.ops._c10d_functional


@pytest.fixture(scope="module")
def env():
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=8)
    install()
    sys.path.insert(0, REFERENCE)
    try:
        import autoparallel.asynctp as asynctp
    finally:
        sys.path.remove(REFERENCE)
    assert sys.modules["autoparallel.asynctp_ops"] is ops
    yield asynctp, dist.group.WORLD.group_name
    dist.destroy_process_group()


def _rewrite(asynctp, fn, specs):
    """Trace ``fn`` on fake CUDA tensors described by (shape, dtype, transposed) and run the pass."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.distributed._symmetric_memory import _test_mode
    from torch.fx.experimental.proxy_tensor import make_fx

    with FakeTensorMode():
        args = []
        for shape, dtype, transposed in specs:
            t = torch.empty(*shape, dtype=dtype, device="cuda")
            args.append(t.t() if transposed else t)
        gm = make_fx(fn, tracing_mode="fake")(*args)
    with _test_mode():
        asynctp.micro_pipeline_tp_pass(gm.graph)
    gm.graph.lint()
    return gm


def _calls(gm, target):
    return [n for n in gm.graph.nodes if n.op == "call_function" and n.target == target]


def _live_targets(gm):
    """Targets of the nodes the output depends on (the pass may leave dead collectives behind)."""
    out = next(n for n in gm.graph.nodes if n.op == "output")
    seen, todo = set(), [out]
    while todo:
        n = todo.pop()
        if n in seen:
            continue
        seen.add(n)
        todo.extend(n.all_input_nodes)
    return {n.target for n in seen if n.op == "call_function"}


def test_last_dim_gather_is_emitted_as_gather_dim_1(env):
    """asynctp.py:767-772 routes a last-dim all-gather (>= 1024 columns per shard) to the fused
    op with gather_dim = 1; the K-split body on the CUDA side takes it from there."""
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(x, w):
        return funcol.all_gather_tensor(x, 1, g) @ w

    gm = _rewrite(asynctp, f, [((512, 1024), BF, False), ((8192, 1024), BF, False)])
    (n,) = _calls(gm, NS.fused_all_gather_matmul.default)
    assert n.args[2] == 1 and n.args[3] == g and n.kwargs.get("return_A") is False
    assert C10D.all_gather_into_tensor.default not in _live_targets(gm)
    # shapes the Meta kernel promises for that call
    _, outs = NS.fused_all_gather_matmul(torch.empty(512, 1024, device="meta", dtype=BF), [torch.empty(8192, 1024, device="meta", dtype=BF)], 1, g, return_A=False)
    assert tuple(outs[0].shape) == (512, 1024)


def test_last_dim_scatter_is_emitted_as_scatter_dim_1(env):
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(h, w):
        return funcol.reduce_scatter_tensor(h @ w, "sum", 1, g)

    gm = _rewrite(asynctp, f, [((512, 1024), BF, False), ((1024, 8192), BF, False)])
    (n,) = _calls(gm, NS.fused_matmul_reduce_scatter.default)
    assert n.args[2:] == ("sum", 1, g)
    assert C10D.reduce_scatter_tensor.default not in _live_targets(gm)
    out = NS.fused_matmul_reduce_scatter(torch.empty(512, 1024, device="meta", dtype=BF), torch.empty(1024, 8192, device="meta", dtype=BF), "sum", 1, g)
    assert tuple(out.shape) == (512, 1024)


def test_avg_reduce_travels_as_reduce_op(env):
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(h, w):
        return funcol.reduce_scatter_tensor(h @ w, "avg", 0, g)

    gm = _rewrite(asynctp, f, [((2048, 1024), BF, False), ((1024, 512), BF, False)])
    (n,) = _calls(gm, NS.fused_matmul_reduce_scatter.default)
    assert n.args[2:] == ("avg", 0, g)
    assert C10D.reduce_scatter_tensor.default not in _live_targets(gm)


def test_gathered_A_is_returned_when_the_graph_uses_it(env):
    """asynctp.py:877-882 clears return_A only when nothing else reads the gathered activation."""
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(x, w):
        a = funcol.all_gather_tensor(x, 0, g)
        return a @ w, a.sum()

    gm = _rewrite(asynctp, f, [((256, 1024), BF, False), ((1024, 512), BF, False)])
    (n,) = _calls(gm, NS.fused_all_gather_matmul.default)
    assert n.kwargs.get("return_A", True) is True
    picked = sorted(u.args[1] for u in n.users if u.target == operator.getitem)
    assert picked == [0, 1]
    assert C10D.all_gather_into_tensor.default not in _live_targets(gm)


def test_transposed_matmul_fusion_uses_a_transposed_view_of_B(env):
    """With ``_ag_transpose_mm_enabled`` (asynctp.py:37, :702-725, :804-840) ``w @ all_gather(x).T``
    becomes ``fused_all_gather_matmul(x, [w.T], 0, g, return_A=True)`` followed by a transpose of the
    product: no new operator, B simply arrives as a K-contiguous view, which the CUDA path reads
    through a K-major descriptor without a copy."""
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(x, w):
        return w @ funcol.all_gather_tensor(x, 0, g).permute(1, 0)

    old = asynctp._ag_transpose_mm_enabled
    asynctp._ag_transpose_mm_enabled = True
    try:
        gm = _rewrite(asynctp, f, [((512, 1024), BF, False), ((256, 1024), BF, False)])
    finally:
        asynctp._ag_transpose_mm_enabled = old
    (n,) = _calls(gm, NS.fused_all_gather_matmul.default)
    assert n.args[2] == 0 and n.kwargs.get("return_A") is True
    (b_node,) = n.args[1]
    assert b_node.target == torch.ops.aten.permute.default and list(b_node.args[1]) == [1, 0]
    assert C10D.all_gather_into_tensor.default not in _live_targets(gm)
    # the operand that reaches the op: [K, N] = [1024, 256] with K contiguous -> "n-major = 0"
    w_t = torch.empty(256, 1024, dtype=BF).permute(1, 0)
    prepared, ldb, n_major = ops._prep_B(w_t)
    assert prepared.data_ptr() == w_t.data_ptr() and ldb == 1024 and not n_major
    # and the final value is the transpose of the op's product
    out = next(n for n in gm.graph.nodes if n.op == "output").args[0]
    assert out.target == torch.ops.aten.clone.default
    assert out.args[0].target == torch.ops.aten.permute.default


def test_transposed_matmul_fusion_is_off_by_default(env):
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env
    assert asynctp._ag_transpose_mm_enabled is False

    def f(x, w):
        return w @ funcol.all_gather_tensor(x, 0, g).permute(1, 0)

    gm = _rewrite(asynctp, f, [((512, 1024), BF, False), ((256, 1024), BF, False)])
    assert _calls(gm, NS.fused_all_gather_matmul.default) == []


def test_rowwise_fp8_all_gather_scaled_mm(env):
    """The pass hands over the gathered row scales (``ROW_WISE_REPLICATED``) and a column-major B."""
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(x8, xs, w8, wscale):
        a = funcol.all_gather_tensor(x8, 0, g)
        s = funcol.all_gather_tensor(xs, 0, g)
        return torch._scaled_mm(a, w8, s, wscale, out_dtype=BF)

    gm = _rewrite(asynctp, f, [((256, 1024), F8, False), ((256, 1), F32, False), ((512, 1024), F8, True), ((1, 512), F32, False)])
    (n,) = _calls(gm, NS.fused_all_gather_scaled_matmul.default)
    A, Bs, A_scale, B_scales, gather_dim, group, biases, result_scales, out_dtypes, fast = n.args
    assert gather_dim == 0 and group == g
    assert len(Bs) == len(B_scales) == 1 and biases == [None] and result_scales == [None]
    assert out_dtypes == [BF] and fast == [False]
    assert tuple(A_scale.meta["val"].shape) == (2048, 1)
    mode = ops._check_and_verify_fp8_all_gather_scale_mode(torch.empty(256, 1024), torch.empty(2048, 1), 0, 8)
    assert mode is ops._ScaleMode.ROW_WISE_REPLICATED
    getitems = [u for u in n.users if u.target == operator.getitem]
    assert [u.args[1] for u in getitems] == [1]  # only the products are used, not the gathered A


def test_rowwise_fp8_scaled_mm_reduce_scatter(env):
    import torch.distributed._functional_collectives as funcol

    asynctp, g = env

    def f(h8, hs, w8, wscale):
        y = torch._scaled_mm(h8, w8, hs, wscale, out_dtype=BF)
        return funcol.reduce_scatter_tensor(y, "sum", 0, g)

    gm = _rewrite(asynctp, f, [((2048, 512), F8, False), ((2048, 1), F32, False), ((1024, 512), F8, True), ((1, 1024), F32, False)])
    (n,) = _calls(gm, NS.fused_scaled_matmul_reduce_scatter.default)
    A, B, A_scale, B_scale, reduce_op, orig_dim, dim_after, group, output_shape = n.args[:9]
    assert (reduce_op, orig_dim, dim_after, group) == ("sum", 0, 0, g)
    assert list(output_shape) == [2048, 1024]
    assert n.args[11] == BF and n.args[12] is False
    assert C10D.reduce_scatter_tensor.default not in _live_targets(gm)
    out = NS.fused_scaled_matmul_reduce_scatter(
        torch.empty(2048, 512, device="meta", dtype=F8), torch.empty(1024, 512, device="meta", dtype=F8).t(),
        torch.empty(2048, 1, device="meta"), torch.empty(1, 1024, device="meta"), "sum", 0, 0, g, [2048, 1024], None, None, BF, False,
    )
    assert tuple(out.shape) == (256, 1024) and out.dtype == BF
