"""World-size-2 CPU (gloo) coverage of the multi-rank host path: the oracle over a live process
group, and the symmetric-workspace bookkeeping (handle exchange, growth, epoch parity) with the
native library replaced by a host-memory fake."""
import ctypes as C

import torch
import torch.distributed as dist

from tests._mp import run_ranks


def _oracle_dist_worker(rank, world):
    from oracle import asynctp_oracle as orc

    shards = [orc.activations(r, 24, 32, torch.float32) for r in range(world)]
    Bs = [orc.weights(7, 32, 16, torch.float32), orc.weights(8, 32, 8, torch.float32)]
    A, outs = orc.all_gather_matmul_dist(shards[rank], Bs, 0)
    A_ref, outs_ref = orc.all_gather_matmul_local(shards, Bs, 0)
    assert torch.equal(A, A_ref)
    for o, r in zip(outs, outs_ref):
        torch.testing.assert_close(o, r, rtol=0, atol=0)
    # 3-D, gather along dim 1
    sh3 = [orc.activations(10 + r, 4 * 6, 32, torch.float32).view(4, 6, 32) for r in range(world)]
    A, outs = orc.all_gather_matmul_dist(sh3[rank], Bs, 1)
    A_ref, outs_ref = orc.all_gather_matmul_local(sh3, Bs, 1)
    assert torch.equal(A, A_ref) and torch.equal(outs[0], outs_ref[0])
    # reduce-scatter, sum and avg
    As = [orc.activations(20 + r, 16, 32, torch.float32) for r in range(world)]
    Ws = [orc.weights(30 + r, 32, 8, torch.float32) for r in range(world)]
    for op in ("sum", "avg"):
        out = orc.matmul_reduce_scatter_dist(As[rank], Ws[rank], op, 0)
        ref = orc.matmul_reduce_scatter_local(As, Ws, op, 0)[rank]
        torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-6)
    # fp8 row-wise, both directions
    xs = [orc.quantize_rowwise(orc.activations(40 + r, 16, 32, torch.float32), 1) for r in range(world)]
    w8, ws8 = orc.quantize_rowwise(orc.weights(50, 32, 24, torch.float32), 0)
    A, (o,) = orc.all_gather_scaled_matmul_dist(xs[rank][0], [w8], xs[rank][1], [ws8], 0, [None], [None], [torch.bfloat16])
    A_ref, (o_ref,) = orc.all_gather_scaled_matmul_local(
        [x[0] for x in xs], [w8], [x[1] for x in xs], [ws8], 0, [None], [None], [torch.bfloat16]
    )
    assert torch.equal(A.view(torch.uint8), A_ref.view(torch.uint8)) and torch.equal(o, o_ref)
    out = orc.scaled_matmul_reduce_scatter_dist(xs[rank][0], w8, xs[rank][1], ws8, "sum", 0, [16, 24], out_dtype=torch.bfloat16)
    ref = orc.scaled_matmul_reduce_scatter_local(
        [x[0] for x in xs], [w8] * world, [x[1] for x in xs], [ws8] * world, "sum", 0, [16, 24], out_dtype=torch.bfloat16
    )[rank]
    torch.testing.assert_close(out.float(), ref.float(), rtol=2 ** -7, atol=1e-3)


def test_oracle_over_gloo_matches_local_form():
    run_ranks(_oracle_dist_worker, 2)


class _FakeNative:
    """apk_symm_* over host memory: 'handles' carry the owner's address, import returns it."""

    def __init__(self):
        self.live = {}
        self.imports = 0

    def apk_symm_alloc(self, nbytes, out_ptr):
        buf = (C.c_uint8 * int(nbytes))()
        addr = C.addressof(buf)
        self.live[addr] = buf
        out_ptr._obj.value = addr
        return 0

    def apk_symm_free(self, ptr):
        self.live.pop(ptr.value, None)
        return 0

    def apk_symm_export(self, ptr, handle):
        handle.raw = int(ptr.value).to_bytes(8, "little") + b"\0" * 56
        return 0

    def apk_symm_import(self, handle, out_ptr):
        self.imports += 1
        out_ptr._obj.value = int.from_bytes(handle.raw[:8], "little") | (1 << 62)  # tagged: a peer mapping
        return 0

    def apk_symm_unimport(self, ptr):
        self.imports -= 1
        return 0

    def apk_last_error(self):
        return b""


def _workspace_worker(rank, world):
    from autoparallel_b200 import _native as nat
    from autoparallel_b200 import symm

    fake = _FakeNative()
    nat.lib = lambda: fake
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
    g = dist.group.WORLD.group_name
    w = symm.get_workspace(g, torch.device("cpu"))
    assert (w.rank, w.world) == (rank, world)
    assert symm.get_workspace(g, torch.device("cpu")) is w
    w.ensure(10_000, 512)
    h = symm.peer_handles(g)
    assert h.data_bytes == 2 * 12288 and h.flag_bytes == symm.FLAG_PAD_BYTES
    # every rank sees every rank's local address, its own untagged and the peers' tagged
    mine = torch.tensor([h.data[rank], h.flags[rank]], dtype=torch.int64)
    everyone = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(everyone, mine)
    for r in range(world):
        tag = 0 if r == rank else (1 << 62)
        assert h.data[r] == int(everyone[r][0]) | tag and h.flags[r] == int(everyone[r][1]) | tag
    assert fake.imports == 2 * (world - 1)
    # no growth when it fits, doubling when it does not
    before = list(h.data)
    w.ensure(12_000, 512)
    assert symm.peer_handles(g).data == before
    w.ensure(13_000, 512)
    assert symm.peer_handles(g).data_bytes == 2 * (2 * 12288) and fake.imports == 2 * (world - 1)
    # epochs advance once per collective and select alternating halves
    c1, c2 = w.next_comm(), w.next_comm()
    assert (c1.epoch, c2.epoch) == (1, 2) and c1.world == world and c1.rank == rank
    assert c1.data[1 - rank] == symm.peer_handles(g).data[1 - rank]
    assert c1.ctrl_bytes >= 512 and c1.timeout_s == symm.DEFAULT_TIMEOUT_S
    # a grown arena comes with a zeroed signal pad: the epoch sequence restarts on every rank
    w.ensure(40_000, 512)
    assert symm.peer_handles(g).data_bytes >= 2 * 40_960
    assert w.next_comm().epoch == 1
    w.ensure(40_000, 512)
    assert w.next_comm().epoch == 2
    symm.shutdown()
    assert fake.imports == 0 and not fake.live


def test_workspace_bookkeeping_over_gloo():
    run_ranks(_workspace_worker, 2)
