"""What the host module hands to the C ABI: shapes, leading dimensions, operand layouts, scale modes
and scratch, checked on CPU tensors with the native library replaced by a recorder."""
import ctypes as C

import pytest
import torch
import torch.distributed as dist

import autoparallel_b200.asynctp_ops as ops
from autoparallel_b200 import _native as nat
from autoparallel_b200 import symm


class _Recorder:
    """Stands in for libapk.so: records the argument structs, computes nothing."""

    def __init__(self):
        self.ag, self.rs = [], []

    def apk_ag_gemm_arena_bytes(self, args, world):
        return 0

    def apk_gemm_rs_arena_bytes(self, args, world):
        return 0

    def apk_ctrl_bytes(self, rows, world):
        return 256

    def apk_ag_gemm(self, comm, args, stream):
        a = nat.ApkAgGemmArgs()
        C.memmove(C.byref(a), args, C.sizeof(a))
        c = nat.ApkComm()
        C.memmove(C.byref(c), comm, C.sizeof(c))
        self.ag.append((c, a))
        return 0

    def apk_gemm_rs(self, comm, args, stream):
        a = nat.ApkGemmRsArgs()
        C.memmove(C.byref(a), args, C.sizeof(a))
        self.rs.append(a)
        return 0

    def apk_last_error(self):
        return b""


@pytest.fixture()
def recorder(monkeypatch):
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=3, world_size=8)
    rec = _Recorder()
    monkeypatch.setattr(nat, "lib", lambda: rec)
    monkeypatch.setattr(ops, "_stream_ptr", lambda device: C.c_void_p(0))
    monkeypatch.setattr(symm.GroupWorkspace, "ensure", lambda self, half, ctrl: None)
    monkeypatch.setattr(symm, "_workspaces", {})
    yield rec, dist.group.WORLD.group_name
    dist.destroy_process_group()


def test_all_gather_matmul_marshalling(recorder):
    rec, g = recorder
    bf = torch.bfloat16
    A = torch.zeros(4, 6, 64, dtype=bf)                      # gather along dim 1 -> rows = 6 * 4
    w_row = torch.zeros(64, 40, dtype=bf)                    # row-major B
    w_t = torch.zeros(24, 64, dtype=bf).t()                  # transposed view: K contiguous
    n = [None, None]
    A_out, outs = ops._ag_gemm_native(A, [w_row, w_t], None, n, n, n, [bf, bf], 1, g, True)
    (c, a), = rec.ag
    assert (c.rank, c.world, c.epoch) == (3, 8, 1)
    assert (a.dtype, a.rows_per_rank, a.K, a.nB, a.lda, a.return_A, a.gather_k) == (nat.APK_BF16, 24, 64, 2, 64, 1, 0)
    assert a.A_gathered and a.a_scale_mode == nat.APK_SCALE_NONE
    assert (a.Bs[0].n_major, a.Bs[0].ldb, a.Bs[0].N, a.Bs[0].ldo) == (1, 40, 40, 40)
    assert (a.Bs[1].n_major, a.Bs[1].ldb, a.Bs[1].N, a.Bs[1].ldo) == (0, 64, 24, 24)
    assert a.Bs[1].B == w_t.data_ptr()                       # no copy for either layout
    assert tuple(A_out.shape) == (4, 48, 64) and [tuple(o.shape) for o in outs] == [(4, 48, 40), (4, 48, 24)]


def test_all_gather_last_dim_marshalling(recorder):
    rec, g = recorder
    bf = torch.bfloat16
    A = torch.zeros(5, 4, 32, dtype=bf)
    B = torch.zeros(32 * 8, 16, dtype=bf)
    A_out, (o,) = ops._ag_gemm_native(A, [B], None, [None], [None], [None], [bf], 2, g, True)
    (_, a), = rec.ag
    assert (a.gather_k, a.rows_per_rank, a.K, a.return_A) == (1, 20, 32, 1)
    assert tuple(A_out.shape) == (5, 4, 256) and tuple(o.shape) == (5, 4, 16)


def test_scaled_all_gather_marshalling(recorder):
    rec, g = recorder
    f8 = torch.float8_e4m3fn
    A = torch.zeros(16, 32, dtype=f8)
    B = torch.zeros(24, 32, dtype=f8).t()
    bias = torch.zeros(24, dtype=torch.bfloat16)
    for scale, mode in ((torch.ones(16, 1), nat.APK_SCALE_VECTOR), (torch.ones(128, 1), nat.APK_SCALE_ROWS_REPLICATED),
                        (torch.tensor(2.0), nat.APK_SCALE_SCALAR)):
        ops._fused_all_gather_scaled_matmul(A, [B], scale, [torch.ones(1, 24)], 0, g, [bias], [torch.tensor(0.5)],
                                            [15], [True])      # 15 = ScalarType of bfloat16
        _, a = rec.ag[-1]
        assert (a.dtype, a.a_scale_mode, a.return_A) == (nat.APK_E4M3, mode, 1)
        op = a.Bs[0]
        assert (op.n_major, op.b_scale_mode, op.out_dtype, op.bias_dtype) == (0, nat.APK_SCALE_VECTOR, nat.APK_BF16, nat.APK_BF16)
        assert op.bias and op.result_scale and op.b_scale
        assert bool(a.A_scale_gathered) == (mode == nat.APK_SCALE_VECTOR)


def test_reduce_scatter_marshalling(recorder):
    rec, g = recorder
    bf = torch.bfloat16
    A = torch.zeros(4, 16, 64, dtype=bf)
    B = torch.zeros(64, 40, dtype=bf)
    out = ops._fused_matmul_reduce_scatter(A, B, "avg", 1, g)          # scatter dim 1: 16 -> 2
    a = rec.rs[-1]
    assert (a.M, a.K, a.reduce_op, a.lda, a.scatter_cols) == (64, 64, nat.APK_REDUCE_AVG, 64, 0)
    assert (a.B.N, a.B.ldo, a.B.n_major) == (40, 40, 1) and tuple(out.shape) == (4, 2, 40)
    out = ops._fused_matmul_reduce_scatter(A, B, "sum", 2, g)          # last dim: columns are scattered
    a = rec.rs[-1]
    assert (a.M, a.scatter_cols, a.B.N, a.B.ldo) == (64, 1, 40, 5) and tuple(out.shape) == (4, 16, 5)
    with pytest.raises(ValueError, match="not divisible"):
        ops._fused_matmul_reduce_scatter(torch.zeros(4, 12, 64, dtype=bf), B, "sum", 1, g)


def test_scaled_reduce_scatter_marshalling(recorder):
    rec, g = recorder
    f8 = torch.float8_e4m3fn
    A = torch.zeros(2, 32, 64, dtype=f8)
    B = torch.zeros(48, 64, dtype=f8).t()
    out = ops._fused_scaled_matmul_reduce_scatter(
        A, B, torch.ones(2, 32, 1), torch.ones(1, 48), "sum", 1, 1, g, [2, 32, 48], None, None, torch.bfloat16, False
    )
    a = rec.rs[-1]
    assert (a.dtype, a.M, a.K, a.a_scale_mode, a.B.b_scale_mode, a.B.n_major) == (
        nat.APK_E4M3, 64, 64, nat.APK_SCALE_VECTOR, nat.APK_SCALE_VECTOR, 0)
    assert tuple(out.shape) == (2, 4, 48) and out.dtype == torch.bfloat16
    with pytest.raises(ValueError, match="leading dims of A_scale"):
        ops._fused_scaled_matmul_reduce_scatter(
            A, B, torch.ones(3, 32, 1), torch.ones(1, 48), "sum", 1, 1, g, [2, 32, 48], None, None, torch.bfloat16, False
        )


def test_more_operands_than_one_launch_takes(recorder):
    """Six Bs (the reference takes any number, autoparallel/asynctp_ops.py:445-454): one fused launch
    for the first four that also leaves the whole gathered A behind, then a local launch (a group of
    one, no epoch) for the rest on that gathered A."""
    rec, g = recorder
    bf = torch.bfloat16
    A = torch.zeros(16, 64, dtype=bf)
    Bs = [torch.zeros(64, 8 * (i + 1), dtype=bf) for i in range(6)]
    n = [None] * 6
    A_out, outs = ops._ag_gemm_native(A, Bs, None, n, n, n, [bf] * 6, 0, g, False)
    (c0, a0), (c1, a1) = rec.ag
    assert A_out is None and [tuple(o.shape) for o in outs] == [(128, 8 * (i + 1)) for i in range(6)]
    assert (c0.world, c0.epoch, a0.nB, a0.rows_per_rank, a0.return_A) == (8, 1, 4, 16, 1)
    assert (c1.world, c1.rank, a1.nB, a1.rows_per_rank, a1.K) == (1, 0, 2, 128, 64)
    assert a1.A_shard == a0.A_gathered and [a1.Bs[i].N for i in range(2)] == [40, 48]
    assert symm.get_workspace(g, A.device).epoch == 1            # the local launch is not a collective


def test_more_operands_with_row_scales(recorder):
    rec, g = recorder
    f8 = torch.float8_e4m3fn
    A = torch.zeros(16, 32, dtype=f8)
    Bs = [torch.zeros(24, 32, dtype=f8).t() for _ in range(5)]
    ops._fused_all_gather_scaled_matmul(A, Bs, torch.ones(16, 1), [torch.ones(1, 24)] * 5, 0, g, [None] * 5, [None] * 5,
                                        [torch.bfloat16] * 5, [False] * 5)
    (_, a0), (c1, a1) = rec.ag
    assert (a0.nB, a0.a_scale_mode) == (4, nat.APK_SCALE_VECTOR)
    # the second launch sees one scale per row of the gathered A: the peers' rows gathered by the kernel, own rows copied in
    assert (c1.world, a1.nB, a1.a_scale_mode, a1.rows_per_rank) == (1, 1, nat.APK_SCALE_ROWS_REPLICATED, 128)
    assert a1.A_scale == a0.A_scale_gathered


def test_empty_inputs_are_not_collectives(recorder):
    """No rows: nothing is launched and the group's epoch does not move (an op that advanced it
    without waiting for its peers would break the arena's two-op reuse distance)."""
    rec, g = recorder
    bf = torch.bfloat16
    A_out, (o,) = ops._ag_gemm_native(torch.zeros(0, 64, dtype=bf), [torch.zeros(64, 8, dtype=bf)], None, [None], [None],
                                      [None], [bf], 0, g, True)
    assert tuple(A_out.shape) == (0, 64) and tuple(o.shape) == (0, 8)
    out = ops._fused_matmul_reduce_scatter(torch.zeros(0, 64, dtype=bf), torch.zeros(64, 8, dtype=bf), "sum", 0, g)
    assert tuple(out.shape) == (0, 8)
    assert not rec.ag and not rec.rs
    assert g not in symm._workspaces or symm._workspaces[g].epoch == 0


def test_float16_operands(recorder):
    """float16 operands go to the same kernels (kind::f16 takes either 16-bit format). With peers a float16
    reduce-scatter is computed with fp32 partials and rounded once at the end."""
    rec, g = recorder
    h = torch.float16
    A_out, (o,) = ops._fused_all_gather_matmul(torch.zeros(16, 64, dtype=h), [torch.zeros(64, 40, dtype=h)], 0, g)
    (_, a), = rec.ag
    assert (a.dtype, a.Bs[0].out_dtype) == (nat.APK_F16, nat.APK_F16) and o.dtype == h and A_out.dtype == h
    out = ops._fused_matmul_reduce_scatter(torch.zeros(64, 64, dtype=h), torch.zeros(64, 40, dtype=h), "sum", 0, g)
    r = rec.rs[-1]
    assert (r.dtype, r.B.out_dtype) == (nat.APK_F16, nat.APK_F32) and out.dtype == h and tuple(out.shape) == (8, 40)
    with pytest.raises(NotImplementedError, match="float16"):
        ops._fused_all_gather_matmul(torch.zeros(16, 64), [torch.zeros(64, 40)], 0, g)     # fp32 operands: no tensor-core format
