"""Symmetric buffers and signal pads, one set per process-group name.

Replaces what the reference obtains from ``get_symm_mem_workspace(group_name, min_size)`` and
``symm_mem.barrier(channel)`` (autoparallel/asynctp_ops.py:61-65, :229-242): a grow-only data
arena that every rank of the group can address on every peer, plus a zero-initialised signal
pad. Memory comes from ``apk_symm_alloc`` (cudaMalloc) and is mapped into the peers with CUDA
IPC handles exchanged through the process group, one process per GPU.

Protocol facts the kernels rely on (kept here because this module owns ``epoch``):

* every collective op on a group increments ``epoch`` by one on every rank (all ranks call in
  the same order, like any collective);
* the data arena is used in two halves selected by ``epoch & 1``; in every op each rank waits
  for a signal that every other rank produces during the same op, so a rank that has reached
  op ``e + 2`` knows that all peers have finished op ``e`` and may overwrite that half;
* flags carry epoch values and are compared with ``>=`` (wrap-safe), so they are never reset;
  when the arena grows, the new signal pad is zero and the epoch restarts from zero with it;
* the epoch reaches the kernel by value, so a collective op must not be recorded into a CUDA
  graph: a replay would carry the recorded epoch, every flag would already satisfy
  ``flag >= epoch`` and the kernel would read data the peers have not written yet.
  ``next_comm()`` therefore refuses to run during stream capture when the group has peers
  (the reference's barriers, autoparallel/asynctp_ops.py:65, :147, are replay-safe; this
  protocol is not, and says so instead of computing garbage). A group of one rank has no
  flags and may be captured.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.distributed.distributed_c10d as c10d

from . import _native as nat

FLAG_PAD_BYTES = 4096 + 4 * nat.APK_MAX_WORLD * 65536  # staged flags + 65536 tile flags per source rank
DEFAULT_TIMEOUT_S = 30.0
# Guard zones in front of and behind the data arena and the signal pad, filled with a pattern at allocation and
# compared in check_guards(): a kernel (local or a peer's, the zones are part of the peer-mapped allocation) that
# writes outside the arena it was given shows up here. Stands in for a memory checker where none can be run.
GUARD_BYTES = 4096
GUARD_WORD = 0x5AFEC0DE   # below 2**31: the same value as a signed 32-bit word


def _capturing() -> bool:
    """True while the current CUDA stream records a graph (False on a machine without CUDA)."""
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class PeerHandles:
    """Peer-mapped addresses of one group: index = rank inside the group."""

    rank: int
    world: int
    data: list[int] = field(default_factory=list)
    flags: list[int] = field(default_factory=list)
    data_bytes: int = 0
    flag_bytes: int = 0


class GroupWorkspace:
    """Arena + signal pad + per-call scratch of one process group on this rank."""

    def __init__(self, group_name: str, device: torch.device):
        self.group_name = group_name
        self.group = c10d._resolve_process_group(group_name)
        self.rank = dist.get_rank(self.group)
        self.world = self.group.size()
        if self.world > nat.APK_MAX_WORLD:
            raise ValueError(f"group {group_name!r} has {self.world} ranks; at most {nat.APK_MAX_WORLD} are supported")
        self.device = device
        self.epoch = 0
        self.timeout_s = DEFAULT_TIMEOUT_S
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.ctrl = torch.zeros(1024, dtype=torch.int32, device=device)
        self.handles = PeerHandles(self.rank, self.world)
        self._local_data = 0        # base addresses of the local allocations (guard zones included)
        self._local_flags = 0
        self._local_sizes = (0, 0)  # usable bytes of the arena and of the pad
        self._imported: list[int] = []

    # ------------------------------------------------------------------ allocation
    def _exchange(self, ptr: int) -> list[int]:
        """All ranks publish the IPC handle of ``ptr``; returns the peer-mapped addresses."""
        L = nat.lib()
        buf = C.create_string_buffer(64)
        nat.check(L.apk_symm_export(C.c_void_p(ptr), buf))
        gathered: list[bytes | None] = [None] * self.world
        dist.all_gather_object(gathered, buf.raw, group=self.group)
        out = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                out.append(ptr)
                continue
            p = C.c_void_p()
            nat.check(L.apk_symm_import(C.create_string_buffer(h, 64), C.byref(p)))
            self._imported.append(p.value)
            out.append(p.value)
        return out

    def _release(self) -> None:
        L = nat.lib()
        for p in self._imported:
            L.apk_symm_unimport(C.c_void_p(p))
        self._imported = []
        if self._local_data:
            L.apk_symm_free(C.c_void_p(self._local_data))
            self._local_data = 0
        if self._local_flags:
            L.apk_symm_free(C.c_void_p(self._local_flags))
            self._local_flags = 0

    def ensure(self, half_bytes: int, ctrl_bytes: int) -> None:
        """Grow the arena so that each half holds ``half_bytes``. Collective when it grows:
        shapes are congruent across ranks, so every rank takes the same decision."""
        if ctrl_bytes > self.ctrl.numel() * 4:
            self.ctrl = torch.zeros(_round_up(ctrl_bytes, 4096) // 4, dtype=torch.int32, device=self.device)
        if self.world == 1:
            return
        need = 2 * _round_up(half_bytes, 4096)
        if need <= self.handles.data_bytes and self._local_flags:
            return
        if _capturing():
            raise RuntimeError("the symmetric workspace cannot grow during CUDA graph capture")
        L = nat.lib()
        # Nobody may still be reading the old arena: drain the device, then meet the peers.
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._release()
        need = max(need, 2 * self.handles.data_bytes)
        with torch.cuda.device(self.device):
            p = C.c_void_p()
            nat.check(L.apk_symm_alloc(need + 2 * GUARD_BYTES, C.byref(p)))
            self._local_data = p.value
            f = C.c_void_p()
            nat.check(L.apk_symm_alloc(FLAG_PAD_BYTES + 2 * GUARD_BYTES, C.byref(f)))
            self._local_flags = f.value
            self._local_sizes = (need, FLAG_PAD_BYTES)
            self._fill_guards()
            # what the kernels see starts behind the leading guard zone, on every rank alike
            self.handles.data = [a + GUARD_BYTES for a in self._exchange(self._local_data)]
            self.handles.flags = [a + GUARD_BYTES for a in self._exchange(self._local_flags)]
        self.handles.data_bytes = need
        self.handles.flag_bytes = FLAG_PAD_BYTES
        # A zero-filled pad starts a new epoch sequence (all ranks grow in the same call, so they
        # agree): flags are compared wrap-safe, which holds only while flag and epoch are less
        # than 2**31 ops apart, and zeros next to an old epoch count need not be.
        self.epoch = 0
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ guard zones and flag sanity
    def _guard_views(self) -> list[torch.Tensor]:
        """The four guard zones of the local allocations as int32 device tensors (empty list before allocation)."""
        out = []
        for base, size in zip((self._local_data, self._local_flags), self._local_sizes):
            if base:
                for addr in (base, base + GUARD_BYTES + size):
                    out.append(_device_int32_view(addr, GUARD_BYTES // 4, self.device))
        return out

    def _fill_guards(self) -> None:
        for v in self._guard_views():
            v.fill_(GUARD_WORD)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def check_guards(self) -> None:
        """Raise if anything was written in front of or behind the arena or the signal pad, or if a 'staged'
        flag holds a value that no op of this group can have written yet (flags only ever carry epochs that
        have been reached: a larger value means a stray write or a confused epoch sequence)."""
        names = ("before the data arena", "behind the data arena", "before the signal pad", "behind the signal pad")
        want = GUARD_WORD
        for name, v in zip(names, self._guard_views()):
            bad = (v != want).nonzero()
            if bad.numel():
                raise RuntimeError(
                    f"group {self.group_name!r}: guard zone {name} was overwritten "
                    f"({bad.numel()} words, first at byte offset {int(bad[0]) * 4})")
        if self._local_flags:
            staged = _device_int32_view(self._local_flags + GUARD_BYTES, 1024, self.device).cpu()
            ahead = ((staged.to(torch.int64) - self.epoch + (1 << 31)) % (1 << 32)) - (1 << 31)   # wrap-safe flag - epoch
            if bool((ahead > 0).any()):
                raise RuntimeError(
                    f"group {self.group_name!r}: a 'staged' flag is {int(ahead.max())} ahead of the group's epoch {self.epoch}")

    # ------------------------------------------------------------------ per call
    def next_comm(self) -> nat.ApkComm:
        """The comm descriptor of the next collective op (advances the epoch)."""
        if self.world > 1 and _capturing():
            raise RuntimeError(
                "the fused async-TP ops cannot be captured into a CUDA graph when the group has peers: the "
                "flag epoch is passed by value and a replay would reuse it (run them outside the graph, "
                "e.g. torch._inductor.config.triton.cudagraphs = False)"
            )
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF
        c = nat.ApkComm()
        c.rank = self.rank
        c.world = self.world
        for r in range(self.world if self.handles.data else 0):
            c.data[r] = self.handles.data[r]
            c.flags[r] = self.handles.flags[r]
        c.data_bytes = self.handles.data_bytes
        c.flag_bytes = self.handles.flag_bytes
        c.ctrl = self.ctrl.data_ptr()
        c.ctrl_bytes = self.ctrl.numel() * 4
        c.status = self.status.data_ptr()
        c.epoch = self.epoch
        c.timeout_s = self.timeout_s
        return c

    def local_comm(self) -> nat.ApkComm:
        """A descriptor for work on this rank alone (a group of one): no peers, no flags, and the
        group's epoch does not move."""
        c = nat.ApkComm()
        c.rank = 0
        c.world = 1
        c.ctrl = self.ctrl.data_ptr()
        c.ctrl_bytes = self.ctrl.numel() * 4
        c.status = self.status.data_ptr()
        c.epoch = self.epoch
        c.timeout_s = self.timeout_s
        return c

    def check_status(self) -> None:
        """Synchronise and raise if a device-side wait timed out since the last check."""
        c = self.next_comm()
        self.epoch = (self.epoch - 1) & 0xFFFFFFFF  # not a collective: give the epoch back
        raw = C.c_uint32(0)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        nat.check(nat.lib().apk_check_status(C.byref(c), C.c_void_p(stream), C.byref(raw)))

    def close(self) -> None:
        if self._local_data or self._local_flags:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.check_guards()
        self._release()
        self._local_sizes = (0, 0)
        self.handles = PeerHandles(self.rank, self.world)


def _device_int32_view(addr: int, n: int, device: torch.device) -> torch.Tensor:
    """`n` int32 words of memory at `addr` as a tensor on `device` (no copy, no ownership)."""
    if device.type == "cpu":   # host-memory stand-ins of the allocator (CPU tests)
        return torch.frombuffer((C.c_int32 * n).from_address(addr), dtype=torch.int32)

    class _Span:   # the CUDA array interface torch understands
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<i4", "data": (addr, False), "version": 2}

    return torch.as_tensor(_Span(), device=device)


_workspaces: dict[str, GroupWorkspace] = {}


def get_workspace(group_name: str, device: torch.device) -> GroupWorkspace:
    """Workspace of ``group_name`` on this rank (created on first use)."""
    ws = _workspaces.get(group_name)
    if ws is None:
        ws = GroupWorkspace(group_name, device)
        _workspaces[group_name] = ws
    return ws


def peer_handles(group_name: str) -> PeerHandles:
    """The group_name -> NVLink peer-handle map: addresses of every rank's arena and pad."""
    if group_name not in _workspaces:
        raise KeyError(f"no symmetric workspace has been created for group {group_name!r}")
    return _workspaces[group_name].handles


def sync_check(group_name: str | None = None) -> None:
    """Raise ``ApkError`` if any fused op on the group(s) hit a device-side timeout."""
    for name, ws in _workspaces.items():
        if group_name is None or name == group_name:
            ws.check_status()
            ws.check_guards()


def shutdown() -> None:
    """Free every workspace (call before destroying the process group)."""
    for ws in _workspaces.values():
        ws.close()
    _workspaces.clear()
