"""Error behaviour of the symmetric workspace (autoparallel_b200/symm.py), on CPU with fakes:
what the reference gets from torch's workspace (growth refused during CUDA-graph capture,
torch/distributed/_symmetric_memory/__init__.py:96-134) and what replaces its barrier
timeouts (a device status word turned into an exception)."""
import ctypes as C

import pytest
import torch
import torch.distributed as dist

from autoparallel_b200 import _native as nat
from autoparallel_b200 import symm


class _Native:
    """Allocator over host memory plus a scriptable apk_check_status."""

    def __init__(self):
        self.live, self.status_raw = {}, 0

    def apk_symm_alloc(self, nbytes, out_ptr):
        buf = (C.c_uint8 * int(nbytes))()
        self.live[C.addressof(buf)] = buf
        out_ptr._obj.value = C.addressof(buf)
        return 0

    def apk_symm_free(self, ptr):
        self.live.pop(ptr.value, None)
        return 0

    def apk_symm_export(self, ptr, handle):
        handle.raw = int(ptr.value).to_bytes(8, "little") + b"\0" * 56
        return 0

    def apk_symm_import(self, handle, out_ptr):
        out_ptr._obj.value = int.from_bytes(handle.raw[:8], "little")
        return 0

    def apk_symm_unimport(self, ptr):
        return 0

    def apk_check_status(self, comm, stream, raw):
        raw._obj.value = self.status_raw
        return nat.APK_ERR_TIMEOUT if self.status_raw else nat.APK_OK

    def apk_last_error(self):
        return b"device wait timed out: peer partial (detail 3)"


@pytest.fixture()
def group(monkeypatch):
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=1, world_size=4)
    fake = _Native()
    monkeypatch.setattr(nat, "lib", lambda: fake)
    monkeypatch.setattr(symm, "_workspaces", {})
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: type("S", (), {"cuda_stream": 0})())
    yield fake, dist.group.WORLD.group_name
    dist.destroy_process_group()


def test_growth_is_refused_during_graph_capture(group, monkeypatch):
    fake, g = group
    w = symm.get_workspace(g, torch.device("cpu"))
    monkeypatch.setattr(symm, "_capturing", lambda: True)
    with pytest.raises(RuntimeError, match="cannot grow during CUDA graph capture"):
        w.ensure(1 << 20, 256)
    assert not fake.live          # nothing was allocated or exchanged


def test_ops_with_peers_refuse_graph_capture(group, monkeypatch):
    """The epoch travels by value, so a replayed graph would satisfy every flag at once and read data the
    peers have not written: next_comm() refuses during capture and leaves the epoch where it was."""
    fake, g = group
    w = symm.get_workspace(g, torch.device("cpu"))
    w.next_comm()
    before = w.epoch
    monkeypatch.setattr(symm, "_capturing", lambda: True)
    with pytest.raises(RuntimeError, match="cannot be captured into a CUDA graph"):
        w.next_comm()
    assert w.epoch == before
    c = w.local_comm()                    # work on this rank alone has no flags and may be captured
    assert (c.world, c.rank, c.epoch) == (1, 0, before) and w.epoch == before


def test_single_rank_group_needs_no_arena(monkeypatch):
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=1)
    try:
        fake = _Native()
        monkeypatch.setattr(nat, "lib", lambda: fake)
        monkeypatch.setattr(symm, "_workspaces", {})
        w = symm.get_workspace(dist.group.WORLD.group_name, torch.device("cpu"))
        w.ensure(1 << 30, 1 << 16)            # only the local counters grow
        assert not fake.live and w.ctrl.numel() * 4 >= 1 << 16
        c = w.next_comm()
        assert (c.world, c.epoch, c.data_bytes) == (1, 1, 0) and not c.data[0]
    finally:
        dist.destroy_process_group()


def test_groups_larger_than_the_kernel_supports_are_rejected(monkeypatch):
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=16)
    try:
        monkeypatch.setattr(symm, "_workspaces", {})
        with pytest.raises(ValueError, match="at most 8"):
            symm.get_workspace(dist.group.WORLD.group_name, torch.device("cpu"))
    finally:
        dist.destroy_process_group()


def test_unknown_group_has_no_peer_handles(group):
    with pytest.raises(KeyError, match="no symmetric workspace"):
        symm.peer_handles("no-such-group")


def test_device_timeout_surfaces_as_an_exception_and_keeps_the_epoch(group):
    fake, g = group
    w = symm.get_workspace(g, torch.device("cpu"))
    w.next_comm()
    before = w.epoch
    symm.sync_check()                     # status word clear: nothing happens
    fake.status_raw = 4 | (3 << 8)        # "peer partial never arrived", detail = source rank 3
    with pytest.raises(nat.ApkError, match="timed out") as e:
        symm.sync_check(g)
    assert e.value.code == nat.APK_ERR_TIMEOUT
    assert w.epoch == before              # reading the status is not a collective


def test_guard_zones_catch_writes_outside_the_arena(group, monkeypatch):
    """The arena and the signal pad sit between guard zones filled with a pattern; anything written there, or a
    'staged' flag that is ahead of the group's epoch, is reported by the next sync_check()."""
    import ctypes as C

    import contextlib

    fake, g = group
    monkeypatch.setattr(torch.cuda, "device", lambda *a, **k: contextlib.nullcontext())
    monkeypatch.setattr(dist, "barrier", lambda *a, **k: None)
    monkeypatch.setattr(dist, "all_gather_object", lambda out, obj, group=None: [out.__setitem__(i, obj) for i in range(len(out))])
    w = symm.get_workspace(g, torch.device("cpu"))
    w.ensure(1 << 16, 256)
    data_base, flags_base = w._local_data, w._local_flags
    assert w.handles.data[w.rank] == data_base + symm.GUARD_BYTES      # kernels start behind the leading zone
    assert w.handles.flags[w.rank] == flags_base + symm.GUARD_BYTES
    w.next_comm()
    w.check_guards()                                                   # untouched: fine
    C.c_uint32.from_address(data_base + symm.GUARD_BYTES + w.handles.data_bytes + 8).value = 7     # one word behind the arena
    with pytest.raises(RuntimeError, match="behind the data arena"):
        w.check_guards()
    C.c_uint32.from_address(data_base + symm.GUARD_BYTES + w.handles.data_bytes + 8).value = symm.GUARD_WORD
    w.check_guards()
    C.c_uint32.from_address(flags_base + symm.GUARD_BYTES + 128).value = w.epoch + 5               # a flag from the future
    with pytest.raises(RuntimeError, match="ahead of the group's epoch"):
        w.check_guards()
    C.c_uint32.from_address(flags_base + symm.GUARD_BYTES + 128).value = w.epoch
    w.check_guards()
