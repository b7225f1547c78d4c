"""The fused ops under inductor, on real GPUs: a tensor-parallel MLP written with functional collectives is
compiled with ``torch.compile``; the micro-pipeline pass rewrites all-gather -> matmul and matmul ->
reduce-scatter into the fused calls (as AutoParallel does from its post-grad hook,
examples/example_llama3.py:224-241), inductor lowers them as fallback kernels with a fixed stride order, and
the compiled function must agree with the eager, unfused one.

AutoParallel's own pass (autoparallel/asynctp.py) is checked unmodified on CPU in tests/test_fx_pass.py; its
sources are not available where the GPU tests run, so this test drives the pass it was forked from,
``torch._inductor.fx_passes.micro_pipeline_tp``, which inserts the same four calls with the same arguments
under torch's namespace, and retargets them (autoparallel_b200.install.retarget_symm_mem_calls).
Two ranks when the machine has two GPUs, otherwise a group of one.
"""
import pytest
import torch

from tests._mp import run_ranks

pytestmark = pytest.mark.gpu

TOL = 1e-2


def _worker(rank, world, with_backward):
    import torch._inductor.config as ic
    import torch.distributed as dist
    import torch.distributed._functional_collectives as funcol
    import torch.nn.functional as F
    from torch._inductor.fx_passes.micro_pipeline_tp import micro_pipeline_tp_pass
    from torch.distributed._symmetric_memory import _test_mode

    import autoparallel_b200.asynctp_ops  # noqa: F401
    from autoparallel_b200 import _native as nat
    from autoparallel_b200 import symm
    from autoparallel_b200.install import retarget_symm_mem_calls

    dev = torch.device("cuda", rank)
    g = dist.group.WORLD.group_name
    ns = torch.ops._ap_symm_mem
    seen = {"retargeted": 0, "ag": 0, "rs": 0}

    def post_pass(graph):
        with _test_mode():      # opens the pass's "symmetric memory enabled for this group" gate; nothing of torch's symmetric memory runs
            micro_pipeline_tp_pass(graph)
        seen["retargeted"] += retarget_symm_mem_calls(graph)
        for n in graph.nodes:
            if n.op == "call_function":
                seen["ag"] += n.target == ns.fused_all_gather_matmul.default
                seen["rs"] += n.target == ns.fused_matmul_reduce_scatter.default

    ic.post_grad_custom_post_pass = post_pass
    ic.fx_graph_cache = False

    ag = funcol.all_gather_tensor_autograd if with_backward else funcol.all_gather_tensor
    rs = funcol.reduce_scatter_tensor_autograd if with_backward else funcol.reduce_scatter_tensor

    def mlp(x, w1, w3, w2):
        a = ag(x, 0, g)
        h = F.silu(a @ w1) * (a @ w3)
        return rs(h @ w2, "sum", 0, g)

    def fresh():
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        x = torch.randn(1024, 1024, device=dev, generator=gen).bfloat16()
        gw = torch.Generator(device=dev).manual_seed(7)       # the weight slices are this rank's own in real TP; here the same on every rank
        w1 = (torch.randn(1024, 512, device=dev, generator=gw) * 0.03).bfloat16()
        w3 = (torch.randn(1024, 512, device=dev, generator=gw) * 0.03).bfloat16()
        w2 = (torch.randn(512, 1024, device=dev, generator=gw) * 0.03).bfloat16()
        ts = [x, w1, w3, w2]
        if with_backward:
            for t in ts:
                t.requires_grad_(True)
        return ts

    def run(fn):
        ts = fresh()
        out = fn(*ts)
        if not with_backward:
            return [out]
        out = funcol.wait_tensor(out) if hasattr(out, "wait") else out
        out.float().square().mean().backward()
        return [out] + [t.grad for t in ts]

    def rel(a, b):
        return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item()

    want = run(mlp)
    before = nat.lib().apk_launch_count()
    got = run(torch.compile(mlp))
    torch.cuda.synchronize()
    launches = nat.lib().apk_launch_count() - before
    symm.sync_check()
    assert seen["retargeted"] >= 2 and seen["ag"] >= 1 and seen["rs"] >= 1, seen
    assert launches >= 2, launches
    for name, a, b in zip(["out", "dx", "dw1", "dw3", "dw2"], got, want):
        assert a.shape == b.shape and a.dtype == b.dtype, name
        e = rel(a, b)
        assert e <= TOL, (name, e)
    if with_backward:
        # the backward graph gathers the output gradient for two consumers: the fused call keeps the gathered A
        assert seen["ag"] >= 2, seen
    symm.shutdown()


def _world():
    return 2 if torch.cuda.device_count() >= 2 else 1


def test_compiled_mlp_forward_uses_the_fused_ops():
    from autoparallel_b200.build import build_native

    build_native()
    run_ranks(_worker, _world(), False, backend="nccl")


def test_compiled_mlp_forward_and_backward():
    from autoparallel_b200.build import build_native

    build_native()
    run_ranks(_worker, _world(), True, backend="nccl")
