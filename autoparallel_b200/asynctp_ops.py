"""Drop-in replacement of AutoParallel's ``autoparallel/asynctp_ops.py``.

Registers the same six ``_ap_symm_mem`` operator schemas (autoparallel/asynctp_ops.py:326-359),
so the unchanged FX pass in ``autoparallel/asynctp.py`` (it inserts
``torch.ops._ap_symm_mem.fused_*`` nodes at :653-674, :717-721, :982-1010) and inductor's
fallback-kernel lowering dispatch to the kernels in libapk.so.

* ``Meta`` kernels are the unfused decompositions (all_gather / reduce_scatter + matmul) that
  define output shapes and dtypes, as in the reference (:672-700, :873-944, :1090-1100, :1242-1290).
* ``CUDA`` kernels validate like the reference, flatten to 2-D with the gather / scatter
  dimension in front, and call ``apk_ag_gemm`` / ``apk_gemm_rs`` through ctypes. There is no
  eager or CPU fallback: an unsupported input raises.

Because a library namespace can be defined only once per process, this module and the
reference's file cannot be imported together; ``autoparallel_b200.install`` puts this module
in ``sys.modules`` under the reference's name.
"""
from __future__ import annotations

import ctypes as C
from enum import Enum
from typing import Any

import torch
import torch.distributed._functional_collectives as funcol
import torch.distributed.distributed_c10d as c10d

from . import _native as nat
from . import symm

# Routes the CUDA kernels to the unfused decompositions (same switch as the reference, :23).
_is_test_mode: bool = False

lib = torch.library.Library("_ap_symm_mem", "DEF")  # noqa: TOR901
lib.define(
    "fused_all_gather_matmul("
    "Tensor A, Tensor[] Bs, int gather_dim, str group_name, *, bool return_A = True) -> (Tensor?, Tensor[])",
    tags=[torch._C.Tag.needs_fixed_stride_order],
)
lib.define(
    "fused_all_gather_scaled_matmul("
    "Tensor A, Tensor[] Bs, Tensor A_scale, Tensor[] B_scales, "
    "int gather_dim, str group_name, "
    "Tensor?[] biases, "
    "Tensor?[] result_scales, "
    "ScalarType?[] out_dtypes, "
    "bool[] use_fast_accum) -> (Tensor, Tensor[])",
    tags=[torch._C.Tag.needs_fixed_stride_order],
)
lib.define(
    "fused_matmul_reduce_scatter(Tensor A, Tensor B, str reduce_op, int scatter_dim, str group_name) -> Tensor",
    tags=[torch._C.Tag.needs_fixed_stride_order],
)
lib.define(
    "fused_scaled_matmul_reduce_scatter("
    "Tensor A, Tensor B, Tensor A_scale, Tensor B_scale, "
    "str reduce_op, int orig_scatter_dim, int scatter_dim_after_maybe_reshape, str group_name, int[]? output_shape, "
    "Tensor? bias = None, "
    "Tensor? result_scale = None, "
    "ScalarType? out_dtype = None, "
    "bool use_fast_accum = False) -> Tensor",
    tags=[torch._C.Tag.needs_fixed_stride_order],
)
lib.define("_low_contention_all_gather(Tensor tensor, str group_name) -> Tensor")
lib.define("_low_contention_reduce_scatter(Tensor tensor, str reduce_op, str group_name) -> Tensor")


class _ScaleMode(Enum):
    UNSCALED = "unscaled"
    TENSOR_WISE = "tensor-wise"
    ROW_WISE_SHARDED = "row-wise-sharded"
    ROW_WISE_REPLICATED = "row-wise-replicated"


def _check_and_verify_fp8_all_gather_scale_mode(
    shard: torch.Tensor, scale: torch.Tensor | None, gather_dim: int, group_size: int
) -> _ScaleMode:
    """Classify ``A_scale`` of an fp8 all-gather (same rules, in the same order, as
    autoparallel/asynctp_ops.py:369-392; a [.., 1] scale whose leading dims equal the shard's is
    taken as row-wise and sharded)."""
    if scale is None:
        return _ScaleMode.UNSCALED
    gathered_shape = list(shard.shape)
    gathered_shape[gather_dim] *= group_size
    if scale.shape[:-1] == shard.shape[:-1] and scale.shape[-1] == 1:
        return _ScaleMode.ROW_WISE_SHARDED
    if scale.numel() == 1:
        return _ScaleMode.TENSOR_WISE
    if list(scale.shape[:-1]) == gathered_shape[:-1]:
        return _ScaleMode.ROW_WISE_REPLICATED
    raise ValueError(
        "Invalid scale shape for fp8 all-gather " f"(shard shape: {shard.shape}, scale shape: {scale.shape})"
    )


# c10 ScalarType enum value -> dtype, for ``ScalarType?[]`` arguments that arrive as ints
# (autoparallel/asynctp_ops.py:1439-1481).
_SCALAR_TYPE_TO_DTYPE = dict(
    enumerate(
        [
            torch.uint8, torch.int8, torch.short, torch.int, torch.int64, torch.half, torch.float, torch.double,
            torch.complex32, torch.complex64, torch.complex128, torch.bool, torch.qint8, torch.quint8, torch.qint32,
            torch.bfloat16, torch.float8_e5m2, torch.float8_e4m3fn, torch.float8_e5m2fnuz, torch.float8_e4m3fnuz,
        ]
    )
)


def _maybe_convert_scalar_types_to_dtypes(scalar_types: list[Any]) -> list[torch.dtype | None]:
    if not all(x is None or isinstance(x, int) for x in scalar_types):
        return scalar_types
    out: list[torch.dtype | None] = []
    for st in scalar_types:
        if st is None:
            out.append(None)
        elif st in _SCALAR_TYPE_TO_DTYPE:
            out.append(_SCALAR_TYPE_TO_DTYPE[st])
        else:
            raise ValueError(f"Unrecognized scalar type {st}")
    return out


def make_contiguous_for_perm(t: torch.Tensor, perm: list[int]) -> torch.Tensor:
    """Restride ``t`` such that ``t.permute(perm)`` is contiguous."""
    inverse = sorted(range(len(perm)), key=perm.__getitem__)
    return t.permute(perm).contiguous().permute(inverse)


def _front_perm(ndim: int, dim: int) -> list[int]:
    return [dim] + [d for d in range(ndim) if d != dim]


def restride_A_shard_for_fused_all_gather_matmul(t: torch.Tensor, gather_dim: int) -> torch.Tensor:
    """Stride order for which ``fused_all_gather_matmul`` needs no input copy."""
    return make_contiguous_for_perm(t, _front_perm(t.dim(), gather_dim))


def restride_A_for_fused_matmul_reduce_scatter(t: torch.Tensor, scatter_dim: int) -> torch.Tensor:
    """Stride order for which ``fused_matmul_reduce_scatter`` needs no input copy."""
    return make_contiguous_for_perm(t, _front_perm(t.dim(), scatter_dim))


# =============================================================================== decompositions
def _all_gather_front(x: torch.Tensor, group_size: int, group_name: str) -> torch.Tensor:
    out = torch.ops._c10d_functional.all_gather_into_tensor(x.contiguous(), group_size, group_name)
    return torch.ops._c10d_functional.wait_tensor(out)


@torch.library.impl(lib, "fused_all_gather_matmul", "Meta")
def _fused_all_gather_matmul_fallback(
    A_shard: torch.Tensor,
    Bs: list[torch.Tensor],
    gather_dim: int,
    group_name: str,
    *,
    return_A: bool = True,
) -> tuple[torch.Tensor | None, list[torch.Tensor]]:
    ws = c10d._get_group_size_by_name(group_name)
    stacked = _all_gather_front(A_shard, ws, group_name)
    if gather_dim == A_shard.ndim - 1:
        A = torch.cat(stacked.chunk(ws), dim=-1)
        outs = [torch.matmul(A, B) for B in Bs]
        return (A if return_A else None), outs
    # rows ordered (rank, gather index): put the rank axis next to gather_dim and merge them.
    A = stacked.view(ws, *A_shard.shape).movedim(gather_dim + 1, 1).flatten(0, 1)
    outs = [torch.matmul(A, B).movedim(0, gather_dim) for B in Bs]
    return (A.movedim(0, gather_dim) if return_A else None), outs


@torch.library.impl(lib, "fused_all_gather_scaled_matmul", "Meta")
def _fused_all_gather_scaled_matmul_fallback(
    A_shard: torch.Tensor,
    Bs: list[torch.Tensor],
    A_scale: torch.Tensor,
    B_scales: list[torch.Tensor],
    gather_dim: int,
    group_name: str,
    biases: list[torch.Tensor | None],
    result_scales: list[torch.Tensor | None],
    out_dtypes: list[torch.dtype | None],
    use_fast_accum: list[bool],
) -> tuple[torch.Tensor, list[torch.Tensor]]:
    out_dtypes = _maybe_convert_scalar_types_to_dtypes(out_dtypes)
    ws = c10d._get_group_size_by_name(group_name)
    A = _all_gather_front(A_shard, ws, group_name)
    A = A.view(ws, *A_shard.shape).movedim(gather_dim + 1, 1).flatten(0, 1)
    mode = _check_and_verify_fp8_all_gather_scale_mode(A_shard, A_scale, gather_dim, ws)
    if mode == _ScaleMode.ROW_WISE_SHARDED:
        shard_scale_shape = A_scale.shape
        A_scale = _all_gather_front(A_scale, ws, group_name)
        A_scale = A_scale.view(ws, *shard_scale_shape).movedim(gather_dim + 1, 1).flatten(0, -2)
    elif mode == _ScaleMode.ROW_WISE_REPLICATED:
        A_scale = A_scale.movedim(gather_dim, 0).flatten(0, -2)
    lead = A.shape[:-1]
    outs = []
    for B, B_scale, bias, rs, od, fast in zip(Bs, B_scales, biases, result_scales, out_dtypes, use_fast_accum):
        C2 = torch.ops.aten._scaled_mm(A.flatten(0, -2), B, A_scale, B_scale, bias, rs, out_dtype=od, use_fast_accum=fast)
        outs.append(C2.unflatten(0, lead).movedim(0, gather_dim))
    return A.movedim(0, gather_dim), outs


@torch.library.impl(lib, "fused_matmul_reduce_scatter", "Meta")
def _fused_matmul_reduce_scatter_fallback(
    A: torch.Tensor, B: torch.Tensor, reduce_op: str, scatter_dim: int, group_name: str
) -> torch.Tensor:
    return funcol.wait_tensor(funcol.reduce_scatter_tensor(A @ B, reduce_op, scatter_dim, group_name))


@torch.library.impl(lib, "fused_scaled_matmul_reduce_scatter", "Meta")
def _fused_scaled_matmul_reduce_scatter_fallback(
    A: torch.Tensor,
    B: torch.Tensor,
    A_scale: torch.Tensor,
    B_scale: torch.Tensor,
    reduce_op: str,
    orig_scatter_dim: int,
    scatter_dim_after_maybe_reshape: int,
    group_name: str,
    output_shape: list[int],
    bias: torch.Tensor | None = None,
    result_scale: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    use_fast_accum: bool = False,
) -> torch.Tensor:
    A_scale = _flat_row_scale(A, A_scale)
    C2 = torch._scaled_mm(A.flatten(0, -2).contiguous(), B, A_scale, B_scale, bias, result_scale, out_dtype, use_fast_accum)
    C2 = C2.view(*output_shape[:-1], B.shape[1])
    return funcol.wait_tensor(funcol.reduce_scatter_tensor(C2, reduce_op, orig_scatter_dim, group_name))


def _flat_row_scale(A: torch.Tensor, A_scale: torch.Tensor) -> torch.Tensor:
    """[.., 1] row-wise scale -> [rows, 1]; a one-element scale passes through."""
    if A_scale.numel() > 1:
        if A_scale.shape[:-1] != A.shape[:-1]:
            raise ValueError(
                "For row-wise scaling, the leading dims of A_scale "
                "must match the leading dims of A "
                f"(A shape: {A.shape}, A_scale shape: {A_scale.shape})"
            )
        return A_scale.flatten(0, -2).contiguous()
    if A_scale.numel() != 1:
        raise ValueError("Invalid A_scale shape " f"(A shape: {A.shape}, A_scale shape: {A_scale.shape})")
    return A_scale


# =============================================================================== native path
_DTYPE_CODE = {torch.bfloat16: nat.APK_BF16, torch.float8_e4m3fn: nat.APK_E4M3, torch.float32: nat.APK_F32, torch.float16: nat.APK_F16}


def _in_dtype_code(t: torch.Tensor, what: str) -> int:
    if t.dtype not in (torch.bfloat16, torch.float16, torch.float8_e4m3fn):
        raise NotImplementedError(
            f"{what}: the sm_100a kernels take bfloat16, float16 or float8_e4m3fn operands, got {t.dtype} "
            "(the tensor cores have no fp32 input format; cast the operands)"
        )
    return _DTYPE_CODE[t.dtype]


def _out_dtype_code(dt: torch.dtype, what: str) -> int:
    if dt not in (torch.bfloat16, torch.float16, torch.float32):
        raise NotImplementedError(f"{what}: output dtype must be bfloat16, float16 or float32, got {dt}")
    return _DTYPE_CODE[dt]


def _aligned(t: torch.Tensor) -> torch.Tensor:
    return t if t.data_ptr() % 16 == 0 else t.clone()


def _prep_B(B: torch.Tensor) -> tuple[torch.Tensor, int, int]:
    """Returns (tensor kept alive, ldb in elements, n_major) for a [K, N] operand without
    copying when it is row-major or a transposed view with a TMA-compatible pitch."""
    es = B.element_size()
    unit = 16 // es
    K, N = B.shape
    if B.stride(1) == 1 and (B.stride(0) % unit == 0 or K == 1) and B.stride(0) >= N and B.data_ptr() % 16 == 0:
        return B, B.stride(0), 1
    if B.stride(0) == 1 and (B.stride(1) % unit == 0 or N == 1) and B.stride(1) >= K and B.data_ptr() % 16 == 0:
        return B, B.stride(1), 0
    Bc = _aligned(B.contiguous())
    return Bc, N, 1


def _fill_operand(
    op: nat.ApkOperand,
    keep: list,
    B: torch.Tensor,
    out: torch.Tensor,
    B_scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    result_scale: torch.Tensor | None,
) -> None:
    Bt, ldb, n_major = _prep_B(B)
    keep.append(Bt)
    op.B = Bt.data_ptr()
    op.ldb = ldb
    op.n_major = n_major
    op.N = B.shape[1]
    op.out = out.data_ptr()
    op.ldo = out.stride(0)
    op.out_dtype = _out_dtype_code(out.dtype, "output")
    if B_scale is not None:
        s = B_scale.to(torch.float32).contiguous().view(-1)
        if s.numel() == 1:
            op.b_scale_mode = nat.APK_SCALE_SCALAR
        elif s.numel() == B.shape[1]:
            op.b_scale_mode = nat.APK_SCALE_VECTOR
        else:
            raise ValueError(f"B_scale must have 1 or {B.shape[1]} elements, got shape {tuple(B_scale.shape)}")
        keep.append(s)
        op.b_scale = s.data_ptr()
    if bias is not None:
        if bias.numel() != B.shape[1]:
            raise ValueError(f"bias must have {B.shape[1]} elements")
        bb = bias.contiguous().view(-1)
        if bb.dtype not in (torch.bfloat16, torch.float32):
            bb = bb.to(torch.float32)
        keep.append(bb)
        op.bias = bb.data_ptr()
        op.bias_dtype = _DTYPE_CODE[bb.dtype]
    if result_scale is not None:
        rs = result_scale.to(torch.float32).contiguous().view(-1)
        if rs.numel() != 1:
            raise ValueError("result_scale must have one element")
        keep.append(rs)
        op.result_scale = rs.data_ptr()


def _stream_ptr(device: torch.device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ag_gemm_native(
    A_shard: torch.Tensor,
    Bs: list[torch.Tensor],
    A_scale: torch.Tensor | None,
    B_scales: list[torch.Tensor | None],
    biases: list[torch.Tensor | None],
    result_scales: list[torch.Tensor | None],
    out_dtypes: list[torch.dtype | None],
    gather_dim: int,
    group_name: str,
    return_A: bool,
) -> tuple[torch.Tensor | None, list[torch.Tensor]]:
    """2-D core shared by the plain and scaled all-gather matmuls
    (counterpart of _fused_all_gather_matmul_impl, autoparallel/asynctp_ops.py:395-530)."""
    if A_shard.dim() < 2:
        raise ValueError("A_shard must be a matrix")
    for B in Bs:
        if B.dim() != 2:
            raise ValueError("B must be a matrix")
    if len(out_dtypes) != len(Bs):
        raise ValueError("len(out_types) must be the same as len(Bs)")
    if gather_dim < 0 or gather_dim >= A_shard.dim():
        raise ValueError("Invalid gather_dim")
    if gather_dim == A_shard.dim() - 1:
        return _ag_gemm_last_dim_native(A_shard, Bs, A_scale, out_dtypes, group_name, return_A)
    if len(Bs) < 1:
        raise ValueError("at least one B operand is needed")
    group = c10d._resolve_process_group(group_name)
    world = group.size()
    dtype_code = _in_dtype_code(A_shard, "A_shard")
    for B in Bs:
        if B.dtype != A_shard.dtype:
            raise ValueError(f"B dtype {B.dtype} differs from A dtype {A_shard.dtype}")
        if B.shape[0] != A_shard.shape[-1]:
            raise ValueError(f"B has {B.shape[0]} rows but A has {A_shard.shape[-1]} columns")

    fronted = A_shard.movedim(gather_dim, 0)
    lead = [world] + list(fronted.shape[:-1])
    A2 = _aligned(fronted.flatten(0, -2).contiguous())
    rows, K = A2.shape
    M = rows * world

    def unflatten(t: torch.Tensor) -> torch.Tensor:
        return t.view(*lead, t.shape[-1]).flatten(0, 1).movedim(0, gather_dim)

    outs = [A2.new_empty((M, B.shape[1]), dtype=od or B.dtype) for B, od in zip(Bs, out_dtypes)]
    need_gathered = world > 1 or return_A
    A_full = A2.new_empty((M, K)) if need_gathered or rows == 0 else None

    if rows == 0:
        # nothing to gather or multiply: no collective takes place, so the group's epoch must not move
        return (unflatten(A_full) if return_A else None), [unflatten(o) for o in outs]

    # One launch multiplies the gathered A with up to APK_MAX_B operands. Further operands (the
    # reference takes any number, autoparallel/asynctp_ops.py:445-454) reuse the gathered A of the
    # first launch as plain local GEMMs, so nothing crosses NVLink twice.
    first = min(len(Bs), nat.APK_MAX_B)
    more = len(Bs) > first
    if more and A_full is None:
        A_full = A2.new_empty((M, K))
    wsp = symm.get_workspace(group_name, A2.device)
    args = nat.ApkAgGemmArgs()
    keep: list = [A2]
    args.dtype = dtype_code
    args.rows_per_rank = rows
    args.K = K
    args.nB = first
    args.A_shard = A2.data_ptr()
    args.lda = K
    args.A_gathered = A_full.data_ptr() if A_full is not None else None
    args.return_A = 1 if (return_A or more) else 0
    for i in range(first):
        _fill_operand(args.Bs[i], keep, Bs[i], outs[i], B_scales[i], biases[i], result_scales[i])

    mode = _check_and_verify_fp8_all_gather_scale_mode(A_shard, A_scale, gather_dim, world)
    if mode == _ScaleMode.TENSOR_WISE:
        s = A_scale.to(torch.float32).contiguous().view(-1)
        keep.append(s)
        args.a_scale_mode = nat.APK_SCALE_SCALAR
        args.A_scale = s.data_ptr()
    elif mode == _ScaleMode.ROW_WISE_SHARDED:
        s = A_scale.movedim(gather_dim, 0).flatten(0, -2).to(torch.float32).contiguous().view(-1)
        gathered_scale = s.new_empty(M)
        keep += [s, gathered_scale]
        args.a_scale_mode = nat.APK_SCALE_VECTOR
        args.A_scale = s.data_ptr()
        args.A_scale_gathered = gathered_scale.data_ptr()
    elif mode == _ScaleMode.ROW_WISE_REPLICATED:
        s = A_scale.movedim(gather_dim, 0).flatten(0, -2).to(torch.float32).contiguous().view(-1)
        keep.append(s)
        args.a_scale_mode = nat.APK_SCALE_ROWS_REPLICATED
        args.A_scale = s.data_ptr()

    L = nat.lib()
    wsp.ensure(L.apk_ag_gemm_arena_bytes(C.byref(args), world), L.apk_ctrl_bytes(rows, world))
    comm = wsp.next_comm()
    nat.check(L.apk_ag_gemm(C.byref(comm), C.byref(args), _stream_ptr(A2.device)))
    if more:
        full_scale = None
        if mode == _ScaleMode.ROW_WISE_SHARDED:
            # the kernel gathered the peers' row scales; add this rank's own rows
            full_scale = gathered_scale
            full_scale[wsp.rank * rows:(wsp.rank + 1) * rows].copy_(s)
        elif mode in (_ScaleMode.TENSOR_WISE, _ScaleMode.ROW_WISE_REPLICATED):
            full_scale = s
        for lo in range(first, len(Bs), nat.APK_MAX_B):
            hi = min(lo + nat.APK_MAX_B, len(Bs))
            _local_gemm(wsp, A_full, Bs[lo:hi], outs[lo:hi], full_scale, B_scales[lo:hi], biases[lo:hi], result_scales[lo:hi])
    A_ret = unflatten(A_full) if return_A else None
    return A_ret, [unflatten(o) for o in outs]


def _local_gemm(
    wsp: "symm.GroupWorkspace",
    A: torch.Tensor,
    Bs: list[torch.Tensor],
    outs: list[torch.Tensor],
    A_scale_full: torch.Tensor | None,
    B_scales: list[torch.Tensor | None],
    biases: list[torch.Tensor | None],
    result_scales: list[torch.Tensor | None],
) -> None:
    """``outs[i] = A @ Bs[i]`` on this rank alone (at most APK_MAX_B operands): the same kernel
    on a group of one. ``A_scale_full`` is one scale or one per row of A."""
    args = nat.ApkAgGemmArgs()
    keep: list = [A]
    args.dtype = _in_dtype_code(A, "A")
    args.rows_per_rank, args.K = A.shape
    args.nB = len(Bs)
    args.A_shard = A.data_ptr()
    args.lda = A.stride(0)
    for i, (B, out) in enumerate(zip(Bs, outs)):
        _fill_operand(args.Bs[i], keep, B, out, B_scales[i], biases[i], result_scales[i])
    if A_scale_full is not None:
        args.a_scale_mode = nat.APK_SCALE_SCALAR if A_scale_full.numel() == 1 else nat.APK_SCALE_ROWS_REPLICATED
        args.A_scale = A_scale_full.data_ptr()
    comm = wsp.local_comm()
    nat.check(nat.lib().apk_ag_gemm(C.byref(comm), C.byref(args), _stream_ptr(A.device)))


def _ag_gemm_last_dim_native(
    A_shard: torch.Tensor,
    Bs: list[torch.Tensor],
    A_scale: torch.Tensor | None,
    out_dtypes: list[torch.dtype | None],
    group_name: str,
    return_A: bool,
) -> tuple[torch.Tensor | None, list[torch.Tensor]]:
    """Gather along the LAST dim: every rank holds a K-slice of A, so
    ``cat(A_shards, -1) @ B == sum_r A_r @ B[r*K:(r+1)*K]``; the kernel accumulates the slices in
    TMEM in the order they arrive (counterpart of _fused_all_gather_matmul_last_gather_dim_impl,
    autoparallel/asynctp_ops.py:602-669)."""
    if A_scale is not None:
        raise NotImplementedError("scaled all-gather matmul along the last dim is not supported (the reference has none either)")
    if len(Bs) < 1:
        raise ValueError("at least one B operand is needed")
    group = c10d._resolve_process_group(group_name)
    world = group.size()
    if A_shard.dtype not in (torch.bfloat16, torch.float16):
        raise NotImplementedError(f"all-gather matmul along the last dim takes bfloat16 or float16 operands, got {A_shard.dtype}")
    lead = list(A_shard.shape[:-1])
    A2 = _aligned(A_shard.flatten(0, -2).contiguous())
    rows, Kc = A2.shape
    for B in Bs:
        if B.dtype != A_shard.dtype:
            raise ValueError(f"B dtype {B.dtype} differs from A dtype {A_shard.dtype}")
        if B.shape[0] != Kc * world:
            raise ValueError(f"B has {B.shape[0]} rows but the gathered A has {Kc * world} columns")
    outs = [A2.new_empty((rows, B.shape[1]), dtype=od or B.dtype) for B, od in zip(Bs, out_dtypes)]
    first = min(len(Bs), nat.APK_MAX_B)
    more = len(Bs) > first
    need_gathered = world > 1 or return_A or more
    stacked = A2.new_empty((world * rows, Kc)) if need_gathered else None   # [world][rows][Kc]
    if rows == 0:
        A_ret = A2.new_empty((*lead, world * Kc)) if return_A else None
        return A_ret, [o.view(*lead, o.shape[-1]) for o in outs]

    wsp = symm.get_workspace(group_name, A2.device)
    args = nat.ApkAgGemmArgs()
    keep: list = [A2]
    args.dtype = _DTYPE_CODE[A_shard.dtype]
    args.rows_per_rank = rows
    args.K = Kc
    args.nB = len(Bs)
    args.A_shard = A2.data_ptr()
    args.lda = Kc
    args.A_gathered = stacked.data_ptr() if stacked is not None else None
    args.return_A = 1 if (return_A or more) else 0
    args.gather_k = 1
    args.nB = first
    for i in range(first):
        _fill_operand(args.Bs[i], keep, Bs[i], outs[i], None, None, None)
    L = nat.lib()
    wsp.ensure(L.apk_ag_gemm_arena_bytes(C.byref(args), world), L.apk_ctrl_bytes(rows, world))
    comm = wsp.next_comm()
    nat.check(L.apk_ag_gemm(C.byref(comm), C.byref(args), _stream_ptr(A2.device)))
    A_cat = None
    if return_A or more:
        # the reference returns cat(shards, -1) (asynctp_ops.py:663-667); here one strided copy
        A_cat = stacked.view(world, rows, Kc).permute(1, 0, 2).reshape(rows, world * Kc)
    for lo in range(first, len(Bs), nat.APK_MAX_B):   # operands beyond one launch's limit: local GEMMs on the gathered A
        hi = min(lo + nat.APK_MAX_B, len(Bs))
        none = [None] * (hi - lo)
        _local_gemm(wsp, A_cat, Bs[lo:hi], outs[lo:hi], None, none, none, none)
    A_ret = A_cat.view(*lead, world * Kc) if return_A else None
    return A_ret, [o.view(*lead, o.shape[-1]) for o in outs]


def _gemm_rs_native(
    A2: torch.Tensor,
    B: torch.Tensor,
    A_scale_rows: torch.Tensor | None,
    B_scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    result_scale: torch.Tensor | None,
    out_dtype: torch.dtype,
    reduce_op: str,
    group_name: str,
    scatter_cols: bool = False,
) -> torch.Tensor:
    """[M, K] @ [K, N] reduced over the group; this rank keeps rows [rank*M/world, (rank+1)*M/world),
    or with ``scatter_cols`` columns [rank*N/world, (rank+1)*N/world) of all rows."""
    group = c10d._resolve_process_group(group_name)
    world = group.size()
    dtype_code = _in_dtype_code(A2, "A")
    if B.dtype != A2.dtype:
        raise ValueError(f"B dtype {B.dtype} differs from A dtype {A2.dtype}")
    M, K = A2.shape
    if B.shape[0] != K:
        raise ValueError(f"B has {B.shape[0]} rows but A has {K} columns")
    if not scatter_cols and M % world != 0:
        raise ValueError(f"the scatter dimension ({M} rows after flattening) is not divisible by the group size {world}")
    A2 = _aligned(A2.contiguous())
    out_shape = (M, B.shape[1] // world) if scatter_cols else (M // world, B.shape[1])
    # Partials cross NVLink as bf16 or fp32. For a float16 result with peers they travel as fp32 (closer to
    # fp64 than the reference's float16 partials, at twice the bytes) and the sum is rounded once at the end.
    via_f32 = out_dtype == torch.float16 and world > 1
    out = A2.new_empty(out_shape, dtype=torch.float32 if via_f32 else out_dtype)
    if M == 0:
        return out.to(out_dtype)   # no rows: no collective takes place and the group's epoch does not move
    wsp = symm.get_workspace(group_name, A2.device)
    args = nat.ApkGemmRsArgs()
    keep: list = [A2]
    args.dtype = dtype_code
    args.M = M
    args.K = K
    args.reduce_op = nat.APK_REDUCE_SUM if reduce_op == "sum" else nat.APK_REDUCE_AVG
    args.A = A2.data_ptr()
    args.lda = K
    args.scatter_cols = 1 if scatter_cols else 0
    _fill_operand(args.B, keep, B, out, B_scale, bias, result_scale)
    if A_scale_rows is not None:
        s = A_scale_rows.to(torch.float32).contiguous().view(-1)
        keep.append(s)
        args.a_scale_mode = nat.APK_SCALE_SCALAR if s.numel() == 1 else nat.APK_SCALE_VECTOR
        args.A_scale = s.data_ptr()
    L = nat.lib()
    wsp.ensure(L.apk_gemm_rs_arena_bytes(C.byref(args), world), 256)
    comm = wsp.next_comm()
    nat.check(L.apk_gemm_rs(C.byref(comm), C.byref(args), _stream_ptr(A2.device)))
    return out.to(torch.float16) if via_f32 else out


def _check_reduce_op(reduce_op: str) -> None:
    if reduce_op not in ("sum", "avg"):
        raise ValueError("reduce_op must be sum or avg")


@torch.library.impl(lib, "fused_all_gather_matmul", "CUDA")
def _fused_all_gather_matmul(
    A_shard: torch.Tensor,
    Bs: list[torch.Tensor],
    gather_dim: int,
    group_name: str,
    *,
    return_A: bool = True,
) -> tuple[torch.Tensor | None, list[torch.Tensor]]:
    """``all_gather_tensor(A_shard, gather_dim, group_name) @ B`` for every B, with the gather
    pipelined inside the GEMM kernel. No input copy is needed when
    ``A_shard.movedim(gather_dim, 0)`` is contiguous."""
    if _is_test_mode:
        return _fused_all_gather_matmul_fallback(A_shard, Bs, gather_dim, group_name, return_A=return_A)
    with torch.profiler.record_function("fused_all_gather_matmul"):
        n = len(Bs)
        return _ag_gemm_native(
            A_shard, Bs, None, [None] * n, [None] * n, [None] * n, [B.dtype for B in Bs], gather_dim, group_name, return_A
        )


@torch.library.impl(lib, "fused_all_gather_scaled_matmul", "CUDA")
def _fused_all_gather_scaled_matmul(
    A_shard: torch.Tensor,
    Bs: list[torch.Tensor],
    A_scale: torch.Tensor,
    B_scales: list[torch.Tensor],
    gather_dim: int,
    group_name: str,
    biases: list[torch.Tensor | None],
    result_scales: list[torch.Tensor | None],
    out_dtypes: list[torch.dtype | None],
    use_fast_accum: list[bool],
) -> tuple[torch.Tensor, list[torch.Tensor]]:
    """fp8 variant: ``_scaled_mm(all_gather(A_shard), B, A_scale, B_scale, ...)`` per B.
    ``A_scale`` may be tensor-wise, row-wise sharded like A, or row-wise replicated.
    Accumulation is always fp32 in TMEM, so ``use_fast_accum`` does not change the result."""
    out_dtypes = _maybe_convert_scalar_types_to_dtypes(out_dtypes)
    if len(biases) != len(Bs):
        raise ValueError("len(biases) must be the same as len(Bs)")
    if len(result_scales) != len(Bs):
        raise ValueError("len(result_scales) must be the same as len(Bs)")
    if len(out_dtypes) != len(Bs):
        raise ValueError("len(out_dtypes) must be the same as len(Bs)")
    if len(use_fast_accum) != len(Bs):
        raise ValueError("len(use_gast_accum_list) must be the same as len(Bs)")
    if len(B_scales) != len(Bs):
        raise ValueError("len(B_scales) must be the same as len(Bs)")
    if _is_test_mode:
        return _fused_all_gather_scaled_matmul_fallback(
            A_shard, Bs, A_scale, B_scales, gather_dim, group_name, biases, result_scales, out_dtypes, use_fast_accum
        )
    with torch.profiler.record_function("fused_all_gather_scaled_matmul"):
        A, outs = _ag_gemm_native(
            A_shard, Bs, A_scale, list(B_scales), list(biases), list(result_scales), list(out_dtypes),
            gather_dim, group_name, True,
        )
        assert A is not None
        return A, outs


@torch.library.impl(lib, "fused_matmul_reduce_scatter", "CUDA")
def _fused_matmul_reduce_scatter(
    A: torch.Tensor, B: torch.Tensor, reduce_op: str, scatter_dim: int, group_name: str
) -> torch.Tensor:
    """``reduce_scatter_tensor(A @ B, reduce_op, scatter_dim, group_name)`` with the partials
    written into the owning rank's memory from the GEMM epilogue. No input copy is needed when
    ``A.movedim(scatter_dim, 0)`` is contiguous."""
    if _is_test_mode:
        return _fused_matmul_reduce_scatter_fallback(A, B, reduce_op, scatter_dim, group_name)
    with torch.profiler.record_function("fused_matmul_reduce_scatter"):
        if A.dim() < 2:
            raise ValueError("A_shard must be a matrix")
        if scatter_dim < 0 or scatter_dim >= A.dim():
            raise ValueError("Invalid gather_dim")
        if B.dim() != 2:
            raise ValueError("B must be a matrix")
        _check_reduce_op(reduce_op)
        world = c10d._resolve_process_group(group_name).size()
        if scatter_dim == A.dim() - 1:
            # rank d receives columns [d*N/world, (d+1)*N/world) of all rows (asynctp_ops.py:1129-1157)
            if B.shape[1] % world != 0:
                raise ValueError(f"B has {B.shape[1]} columns, not divisible by the group size {world}")
            out = _gemm_rs_native(A.flatten(0, -2), B, None, None, None, None, A.dtype, reduce_op, group_name, scatter_cols=True)
            return out.view(*A.shape[:-1], B.shape[1] // world)
        fronted = A.movedim(scatter_dim, 0)
        lead = list(fronted.shape[:-1])
        if lead[0] % world != 0:
            raise ValueError(f"dim {scatter_dim} of A ({lead[0]}) is not divisible by the group size {world}")
        lead[0] //= world
        out = _gemm_rs_native(fronted.flatten(0, -2), B, None, None, None, None, A.dtype, reduce_op, group_name)
        return out.view(*lead, B.shape[1]).movedim(0, scatter_dim)


@torch.library.impl(lib, "fused_scaled_matmul_reduce_scatter", "CUDA")
def _fused_scaled_matmul_reduce_scatter(
    A: torch.Tensor,
    B: torch.Tensor,
    A_scale: torch.Tensor,
    B_scale: torch.Tensor,
    reduce_op: str,
    orig_scatter_dim: int,
    scatter_dim_after_maybe_reshape: int,
    group_name: str,
    output_shape: list[int],
    bias: torch.Tensor | None = None,
    result_scale: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    use_fast_accum: bool = False,
) -> torch.Tensor:
    """fp8 variant of ``fused_matmul_reduce_scatter``: every rank's ``_scaled_mm`` partial
    (scales, bias and result scale applied, rounded to ``out_dtype``) is reduced over the group
    and scattered along ``orig_scatter_dim`` of ``output_shape``."""
    if _is_test_mode:
        return _fused_scaled_matmul_reduce_scatter_fallback(
            A, B, A_scale, B_scale, reduce_op, orig_scatter_dim, scatter_dim_after_maybe_reshape, group_name,
            output_shape, bias, result_scale, out_dtype, use_fast_accum,
        )
    with torch.profiler.record_function("fused_scaled_matmul_reduce_scatter"):
        if A.dim() < 2:
            raise ValueError("A_shard must be a matrix")
        if scatter_dim_after_maybe_reshape < 0 or scatter_dim_after_maybe_reshape >= A.dim():
            raise ValueError("Invalid scatter dim for 2D tensor input to scaled_mm")
        if orig_scatter_dim < 0 or orig_scatter_dim >= len(output_shape):
            raise ValueError("Invalid scatter dim for 3D+ output tensor")
        if B.dim() != 2:
            raise ValueError("B must be a matrix")
        _check_reduce_op(reduce_op)
        if A_scale is None:
            raise ValueError("A_scale cannot be none for scaled_mm")
        out_dtype = _maybe_convert_scalar_types_to_dtypes([out_dtype])[0]
        world = c10d._resolve_process_group(group_name).size()
        sd = scatter_dim_after_maybe_reshape
        fronted = A.movedim(sd, 0)
        lead = list(fronted.shape[:-1])
        if lead[0] % world != 0:
            raise ValueError(f"dim {sd} of A ({lead[0]}) is not divisible by the group size {world}")
        lead[0] //= world
        if A_scale.numel() > 1:
            if A_scale.shape[:-1] != A.shape[:-1]:
                raise ValueError(
                    "For row-wise scaling, the leading dims of A_scale "
                    "must match the leading dims of A "
                    f"(A shape: {A.shape}, A_scale shape: {A_scale.shape})"
                )
            scale_rows = A_scale.movedim(sd, 0).contiguous().flatten(0, -2)
        else:
            scale_rows = A_scale
        out = _gemm_rs_native(
            fronted.flatten(0, -2), B, scale_rows, B_scale, bias, result_scale, out_dtype or A.dtype, reduce_op, group_name
        )
        final_shape = list(output_shape)
        final_shape[-1] = B.shape[1]
        final_shape[orig_scatter_dim] //= world
        return out.view(*lead, B.shape[1]).movedim(0, sd).reshape(final_shape)


@torch.library.impl(lib, "_low_contention_all_gather", "Meta")
def _low_contention_all_gather_meta(tensor: torch.Tensor, group_name: str) -> torch.Tensor:
    ws = c10d._get_group_size_by_name(group_name)
    return tensor.new_empty(tensor.shape[0] * ws, *tensor.shape[1:])


@torch.library.impl(lib, "_low_contention_reduce_scatter", "Meta")
def _low_contention_reduce_scatter_meta(tensor: torch.Tensor, reduce_op: str, group_name: str) -> torch.Tensor:
    ws = c10d._get_group_size_by_name(group_name)
    return tensor.unflatten(0, (ws, -1)).mean(dim=0)


@torch.library.impl(lib, "_low_contention_all_gather", "CUDA")
def _low_contention_all_gather(tensor: torch.Tensor, group_name: str) -> torch.Tensor:
    """``all_gather_tensor(tensor, 0, group_name)`` as one copy kernel over the NVLink peer mappings
    (counterpart of autoparallel/asynctp_ops.py:1524-1610; any dtype, the shard's bytes must be a
    multiple of 16)."""
    world = c10d._resolve_process_group(group_name).size()
    x = _aligned(tensor.contiguous())
    out = x.new_empty((x.shape[0] * world, *x.shape[1:]))
    nbytes = x.numel() * x.element_size()
    if nbytes == 0:
        return out
    wsp = symm.get_workspace(group_name, x.device)
    wsp.ensure(nbytes if world > 1 else 0, 256)
    comm = wsp.next_comm()
    nat.check(nat.lib().apk_all_gather(C.byref(comm), C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), nbytes, _stream_ptr(x.device)))
    return out


@torch.library.impl(lib, "_low_contention_reduce_scatter", "CUDA")
def _low_contention_reduce_scatter(tensor: torch.Tensor, reduce_op: str, group_name: str) -> torch.Tensor:
    """``reduce_scatter_tensor(tensor, reduce_op, 0, group_name)`` with the parts stored straight into
    the owning peers' arenas and summed in fp32 there (counterpart of
    autoparallel/asynctp_ops.py:1613-1702; bfloat16 or float32)."""
    _check_reduce_op(reduce_op)
    world = c10d._resolve_process_group(group_name).size()
    if tensor.dtype not in (torch.bfloat16, torch.float32):
        raise NotImplementedError(f"_low_contention_reduce_scatter takes bfloat16 or float32, got {tensor.dtype}")
    if tensor.shape[0] % world != 0:
        raise ValueError(f"dim 0 ({tensor.shape[0]}) is not divisible by the group size {world}")
    x = _aligned(tensor.contiguous())
    out = x.new_empty((x.shape[0] // world, *x.shape[1:]))
    nbytes = out.numel() * out.element_size()
    if nbytes == 0:
        return out
    wsp = symm.get_workspace(group_name, x.device)
    wsp.ensure(nbytes * world if world > 1 else 0, 256)
    comm = wsp.next_comm()
    nat.check(nat.lib().apk_reduce_scatter(
        C.byref(comm), C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), nbytes, _DTYPE_CODE[x.dtype],
        nat.APK_REDUCE_SUM if reduce_op == "sum" else nat.APK_REDUCE_AVG, _stream_ptr(x.device)))
    return out
