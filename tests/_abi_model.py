"""An executable model of what include/apk.h promises, on host memory. TEST INFRASTRUCTURE ONLY.

``ModelLib`` stands in for libapk.so in CPU tests of the host module: it takes the very argument
structs the host code builds (raw addresses, leading dimensions, layout and scale-mode codes),
interprets them as the header documents them and computes the result with torch on the CPU;
the exchange between ranks, which the real kernels do over NVLink peer mappings, goes through
the test's gloo process group. It follows the kernels' arithmetic where the header fixes it:
fp32 accumulation, ``(acc * a_scale * b_scale + bias) * result_scale``, and in the reduce-scatter
the peers' partials rounded to the output type while the local partial stays fp32, one rounding
after the sum.

With it, the host path (argument checks, movedim / flatten / unflatten, scale handling, output
shapes, workspace growth, epochs) runs end to end without a GPU and can be compared with the
reference's own outputs in tests/golden/. It says nothing about the CUDA kernels: those are
compared with the oracle through the same ABI by the gpu tests.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from autoparallel_b200 import _native as nat

_IN = {nat.APK_BF16: torch.bfloat16, nat.APK_E4M3: torch.float8_e4m3fn, nat.APK_F16: torch.float16}
_OUT = {nat.APK_BF16: torch.bfloat16, nat.APK_F32: torch.float32, nat.APK_F16: torch.float16}


def _bytes(addr: int, nbytes: int) -> torch.Tensor:
    return torch.frombuffer((C.c_uint8 * nbytes).from_address(addr), dtype=torch.uint8)


def _strided(addr: int, rows: int, cols: int, row_stride: int, col_stride: int, dtype: torch.dtype) -> torch.Tensor:
    """[rows, cols] view of host memory at ``addr`` with strides in elements."""
    span = (rows - 1) * row_stride + (cols - 1) * col_stride + 1
    flat = _bytes(addr, span * dtype.itemsize).view(dtype)
    return torch.as_strided(flat, (rows, cols), (row_stride, col_stride))


def _floats(addr: int, n: int) -> torch.Tensor:
    return _bytes(addr, 4 * n).view(torch.float32)


def _struct(ref):
    """The ctypes structure behind a ``byref(...)`` argument."""
    return ref._obj


def _all_gather(t: torch.Tensor, world: int) -> list[torch.Tensor]:
    """Every rank's ``t`` (moved as bytes: gloo has no fp8)."""
    mine = t.contiguous().view(torch.uint8).flatten()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    return [p.view(t.dtype).view(t.shape) for p in parts]


class ModelLib:
    def __init__(self):
        self.live: dict[int, object] = {}
        self.calls: list[str] = []

    # ---------------------------------------------------------------- allocator (host memory)
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
        out_ptr._obj.value = int.from_bytes(handle.raw[:8], "little")   # never dereferenced by the model
        return 0

    def apk_symm_unimport(self, ptr):
        return 0

    def apk_ag_gemm_arena_bytes(self, args, world):
        a = _struct(args)
        return a.rows_per_rank * a.K * _IN[a.dtype].itemsize + 4 * a.rows_per_rank if world > 1 else 0

    def apk_gemm_rs_arena_bytes(self, args, world):
        a = _struct(args)
        return 4 * a.M * a.B.N if world > 1 else 0

    def apk_ctrl_bytes(self, rows, world):
        return 256 + 4 * ((rows + 127) // 128) * max(world, 1)

    def apk_last_error(self):
        return b"model"

    # ---------------------------------------------------------------- operands
    @staticmethod
    def _B(op, K: int, n_cols: int, dtype: torch.dtype) -> torch.Tensor:
        if op.n_major:
            return _strided(op.B, K, n_cols, op.ldb, 1, dtype)
        return _strided(op.B, K, n_cols, 1, op.ldb, dtype)

    @staticmethod
    def _epilogue(acc: torch.Tensor, a_scale, op, cols: slice | None = None) -> torch.Tensor:
        """fp32 [rows, N] -> scaled fp32, in the kernel's order of operations."""
        n = acc.shape[1]
        if a_scale is not None:
            acc = acc * a_scale
        if op.b_scale_mode == nat.APK_SCALE_SCALAR:
            acc = acc * _floats(op.b_scale, 1)
        elif op.b_scale_mode == nat.APK_SCALE_VECTOR:
            acc = acc * _floats(op.b_scale, n).view(1, n)
        if op.bias:
            bias_dtype = _OUT[op.bias_dtype]
            acc = acc + _bytes(op.bias, n * bias_dtype.itemsize).view(bias_dtype).float().view(1, n)
        if op.result_scale:
            acc = acc * _floats(op.result_scale, 1)
        return acc

    # ---------------------------------------------------------------- all-gather -> matmul
    def apk_ag_gemm(self, comm, args, stream):
        c, a = _struct(comm), _struct(args)
        self.calls.append("ag_gemm")
        world, rank, rows, K = c.world, c.rank, a.rows_per_rank, a.K
        dtype = _IN[a.dtype]
        assert a.lda == K or (world == 1 and not a.return_A)
        shard = _strided(a.A_shard, rows, K, a.lda, 1, dtype)
        shards = _all_gather(shard, world) if world > 1 else [shard]
        if a.A_gathered:
            full = _strided(a.A_gathered, world * rows, K, K, 1, dtype)   # gather_k: [world][rows][K], same bytes
            for r, s in enumerate(shards):
                if r != rank or a.return_A:
                    full[r * rows:(r + 1) * rows].view(torch.uint8).copy_(s.view(torch.uint8))
        a_scale = None
        if a.a_scale_mode == nat.APK_SCALE_SCALAR:
            a_scale = _floats(a.A_scale, 1)
        elif a.a_scale_mode == nat.APK_SCALE_VECTOR:
            own = _floats(a.A_scale, rows)
            parts = _all_gather(own, world) if world > 1 else [own]
            a_scale = torch.cat(parts).view(-1, 1)
            if world > 1:
                assert a.A_scale_gathered, "A_scale_gathered is required"
                _floats(a.A_scale_gathered, world * rows).copy_(a_scale.view(-1))
        elif a.a_scale_mode == nat.APK_SCALE_ROWS_REPLICATED:
            a_scale = _floats(a.A_scale, world * rows).view(-1, 1)
        for i in range(a.nB):
            op = a.Bs[i]
            if a.gather_k:
                B = self._B(op, K * world, op.N, dtype).float()
                acc = sum(shards[r].float() @ B[r * K:(r + 1) * K] for r in range(world))
                out_rows = rows
            else:
                acc = torch.cat([s.float() for s in shards]) @ self._B(op, K, op.N, dtype).float()
                out_rows = world * rows
            acc = self._epilogue(acc, a_scale, op)
            out_dtype = _OUT[op.out_dtype]
            _strided(op.out, out_rows, op.N, op.ldo, 1, out_dtype).copy_(acc.to(out_dtype))
        return 0

    # ---------------------------------------------------------------- matmul -> reduce-scatter
    def apk_gemm_rs(self, comm, args, stream):
        c, a = _struct(comm), _struct(args)
        self.calls.append("gemm_rs")
        world, rank, M, K = c.world, c.rank, a.M, a.K
        dtype = _IN[a.dtype]
        op = a.B
        A = _strided(a.A, M, K, a.lda, 1, dtype).float()
        acc = A @ self._B(op, K, op.N, dtype).float()
        a_scale = None
        if a.a_scale_mode == nat.APK_SCALE_SCALAR:
            a_scale = _floats(a.A_scale, 1)
        elif a.a_scale_mode in (nat.APK_SCALE_VECTOR, nat.APK_SCALE_ROWS_REPLICATED):
            a_scale = _floats(a.A_scale, M).view(-1, 1)
        partial = self._epilogue(acc, a_scale, op)
        out_dtype = _OUT[op.out_dtype]
        partials = _all_gather(partial, world) if world > 1 else [partial]
        if a.scatter_cols:
            w = op.N // world
            mine = [p[:, rank * w:(rank + 1) * w] for p in partials]
            out = _strided(op.out, M, w, op.ldo, 1, out_dtype)
        else:
            r = M // world
            mine = [p[rank * r:(rank + 1) * r] for p in partials]
            out = _strided(op.out, r, op.N, op.ldo, 1, out_dtype)
        total = mine[rank].clone()
        for src in range(world):
            if src != rank:
                total += mine[src].to(out_dtype).float()     # what a peer sends is already rounded
        if a.reduce_op == nat.APK_REDUCE_AVG:
            total = total * (1.0 / world)
        out.copy_(total.to(out_dtype))
        return 0

    # ---------------------------------------------------------------- stand-alone collectives
    def apk_all_gather(self, comm, shard, out, nbytes, stream):
        c = _struct(comm)
        self.calls.append("all_gather")
        parts = _all_gather(_bytes(shard.value, nbytes), c.world) if c.world > 1 else [_bytes(shard.value, nbytes)]
        _bytes(out.value, nbytes * c.world).copy_(torch.cat(parts))
        return 0

    def apk_reduce_scatter(self, comm, inp, out, out_bytes, dtype, reduce_op, stream):
        c = _struct(comm)
        self.calls.append("reduce_scatter")
        dt = _OUT[dtype]
        mine = _bytes(inp.value, out_bytes * c.world).view(dt).float()
        parts = _all_gather(mine, c.world) if c.world > 1 else [mine]
        n = out_bytes // dt.itemsize
        total = sum(p[c.rank * n:(c.rank + 1) * n] for p in parts)
        if reduce_op == nat.APK_REDUCE_AVG:
            total = total / c.world
        _bytes(out.value, out_bytes).view(dt).copy_(total.to(dt))
        return 0
