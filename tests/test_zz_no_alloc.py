"""apk_ag_gemm_static: the all-gather matmul for callers that cannot allocate device memory
(a runtime whose pool already owns the whole GPU, or a path where cudaMalloc is forbidden
because it may synchronise the device). Its scratch - per-call counters, the gathered copy of A,
the gathered row scales - is one fixed array inside the library.

The test drives rank 0 of a two-rank group on a single GPU: the "peer" is a second buffer on the
same device that already holds rank 1's staged shard, and rank 1's "staged" flag is set
beforehand, so the kernel's pull, its counters and its gathered buffers are all exercised
without a second process. The new entry point must give the same bits as apk_ag_gemm on two
calls in a row (the two calls use the two halves of the symmetric arena), and both must agree
with the CPU oracle. This file sorts last so that a run that stops at the first failure has
already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

FLAG_STRIDE = 32  # u32 words between two ranks' staged flags in the signal pad


def _round_up(x, a):
    return (x + a - 1) // a * a


class _TwoRankHarness:
    """Buffers of rank 0 and of a pre-staged rank 1 on one device."""

    def __init__(self, nat, rows, K, fp8):
        from oracle import asynctp_oracle as orc

        self.nat, self.rows, self.K, self.fp8 = nat, rows, K, fp8
        dev = "cuda"
        xs = [orc.activations(r, rows, K, torch.float32) for r in range(2)]
        if fp8:
            q = [orc.quantize_rowwise(x, 1) for x in xs]
            self.shards = [a.to(dev) for a, _ in q]
            self.scales = [s.view(-1).contiguous().to(dev) for _, s in q]
        else:
            self.shards = [x.to(torch.bfloat16).to(dev) for x in xs]
            self.scales = None
        es = 1 if fp8 else 2
        chunk = rows * K * es
        self.scale_off = _round_up(chunk, 256)
        self.half = _round_up(self.scale_off + _round_up(rows * 4, 256), 4096)
        self.data = [torch.zeros(2 * self.half, dtype=torch.uint8, device=dev) for _ in range(2)]
        for h in range(2):  # rank 1 has staged its shard (and scales) in both halves
            base = h * self.half
            self.data[1][base: base + chunk] = self.shards[1].view(torch.uint8).view(-1)
            if fp8:
                self.data[1][base + self.scale_off: base + self.scale_off + rows * 4] = self.scales[1].view(torch.uint8)
        self.flags = [torch.zeros(16384, dtype=torch.int32, device=dev) for _ in range(2)]
        self.flags[0][1 * FLAG_STRIDE] = 1000  # "rank 1 staged" for every epoch used here
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.ctrl = torch.zeros(4096, dtype=torch.int32, device=dev)

    def comm(self, epoch, with_ctrl):
        nat = self.nat
        c = nat.ApkComm()
        c.rank, c.world = 0, 2
        for r in range(2):
            c.data[r] = self.data[r].data_ptr()
            c.flags[r] = self.flags[r].data_ptr()
        c.data_bytes, c.flag_bytes = 2 * self.half, self.flags[0].numel() * 4
        if with_ctrl:
            c.ctrl, c.ctrl_bytes = self.ctrl.data_ptr(), self.ctrl.numel() * 4
        c.status, c.epoch, c.timeout_s = self.status.data_ptr(), epoch, 5.0
        return c


def _args(nat, h, B, out, b_scale, gathered, scale_gathered):
    a = nat.ApkAgGemmArgs()
    a.dtype = nat.APK_E4M3 if h.fp8 else nat.APK_BF16
    a.rows_per_rank, a.K, a.nB = h.rows, h.K, 1
    a.A_shard, a.lda = h.shards[0].data_ptr(), h.K
    op = a.Bs[0]
    N = B.shape[1]
    op.B, op.N = B.data_ptr(), N
    if B.stride(1) == 1:
        op.ldb, op.n_major = B.stride(0), 1
    else:
        op.ldb, op.n_major = B.stride(1), 0
    op.out, op.ldo, op.out_dtype = out.data_ptr(), N, nat.APK_BF16
    if h.fp8:
        op.b_scale, op.b_scale_mode = b_scale.data_ptr(), nat.APK_SCALE_VECTOR
        a.A_scale, a.a_scale_mode = h.scales[0].data_ptr(), nat.APK_SCALE_VECTOR
        a.A_scale_gathered = scale_gathered.data_ptr() if scale_gathered is not None else None
    a.A_gathered = gathered.data_ptr() if gathered is not None else None
    a.return_A = 0
    return a


@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8_rowwise"])
def test_static_scratch_entry_matches_regular_entry(fp8):
    from autoparallel_b200 import _native as nat
    from autoparallel_b200.build import build_native
    from oracle import asynctp_oracle as orc

    build_native()
    L = nat.lib()
    torch.cuda.set_device(0)
    rows, K, N = 640, 512, 264
    h = _TwoRankHarness(nat, rows, K, fp8)
    w = orc.weights(7, K, N, torch.float32)
    if fp8:
        b8, sb = orc.quantize_rowwise(w, 0)
        B = b8.cuda().t().contiguous().t()
        b_scale = sb.view(-1).contiguous().cuda()
        ref64 = (torch.cat([s.cpu().double() * sc.cpu().double().view(-1, 1) for s, sc in zip(h.shards, h.scales)])
                 @ (b8.double() * sb.double()))
        tol = 3e-2
    else:
        B = w.to(torch.bfloat16).cuda()
        b_scale = None
        ref64 = torch.cat([s.cpu().double() for s in h.shards]) @ B.cpu().double()
        tol = 1e-2
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    raw = C.c_uint32(0)
    M = 2 * rows
    for epoch in (1, 2):  # two calls in a row: the second uses the other half of the arena
        out_regular = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        out_static = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        gathered = torch.empty(M, K, dtype=h.shards[0].dtype, device="cuda")
        scale_gathered = torch.empty(M, dtype=torch.float32, device="cuda") if fp8 else None

        c = h.comm(epoch, with_ctrl=True)
        a = _args(nat, h, B, out_regular, b_scale, gathered, scale_gathered)
        assert L.apk_ag_gemm(C.byref(c), C.byref(a), stream) == nat.APK_OK, L.apk_last_error()
        assert L.apk_check_status(C.byref(c), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()

        c = h.comm(epoch, with_ctrl=False)  # no ctrl, no gathered buffers: the library's own scratch
        a = _args(nat, h, B, out_static, b_scale, None, None)
        assert L.apk_ag_gemm_static(C.byref(c), C.byref(a), stream) == nat.APK_OK, L.apk_last_error()
        assert L.apk_check_status(C.byref(c), stream, C.byref(raw)) == nat.APK_OK, L.apk_last_error()

        assert not torch.isnan(out_static).any()
        assert torch.equal(out_static, out_regular)
        assert orc.rel_fro_error(out_static, ref64) <= tol
        # the regular call really gathered rank 1's rows through the same path
        assert torch.equal(gathered[rows:].view(torch.uint8), h.shards[1].view(torch.uint8))


def test_static_scratch_entry_rejects_oversize():
    from autoparallel_b200 import _native as nat
    from autoparallel_b200.build import build_native

    build_native()
    L = nat.lib()
    torch.cuda.set_device(0)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    c = nat.ApkComm()
    c.rank, c.world, c.status, c.epoch = 0, 2, status.data_ptr(), 1
    for r in range(2):
        c.data[r] = dummy.data_ptr()
        c.flags[r] = dummy.data_ptr()
    a = nat.ApkAgGemmArgs()
    a.dtype, a.rows_per_rank, a.K, a.nB = nat.APK_BF16, 4096, 4096, 1  # gathered A = 64 MiB > 32 MiB
    before = L.apk_launch_count()
    assert L.apk_ag_gemm_static(C.byref(c), C.byref(a), None) == nat.APK_ERR_SIZE
    assert b"fixed scratch holds" in L.apk_last_error()
    assert L.apk_launch_count() == before
