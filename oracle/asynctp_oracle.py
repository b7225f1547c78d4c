"""CPU oracle for the async-TP fused ops. TEST INFRASTRUCTURE ONLY.

This file restates, on CPU tensors, the unfused decompositions that AutoParallel names as the
semantics of its fused ops (the ``Meta`` kernels of autoparallel/asynctp_ops.py). It is imported
only by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of ``bench.py``;
nothing in ``autoparallel_b200`` imports it and the product never computes through it.

Pinning: the reference's own tests hold no vector for this path. The oracle is pinned against
outputs of the reference's fallbacks themselves (fixtures in ``tests/golden/``):

* ``tests/golden/make_golden.py``, two gloo ranks on CPU: all-gather-matmul (every gather_dim,
  return_A), matmul-reduce-scatter (sum / avg, every scatter_dim) and the scaled
  matmul-reduce-scatter with tensor-wise scales;
* ``tests/golden/make_golden_fp8.py``, two ranks over torch's in-process threaded process group
  (gloo cannot move fp8): the scaled all-gather-matmul with tensor-wise scales on stock torch, and,
  with a CPU stand-in for the row-wise ``aten::_scaled_mm`` that CPU torch lacks, the reference's
  handling of row-wise sharded / replicated scales and the row-wise scaled reduce-scatter.

Parity is UNPINNED by a reference run for one part only: the row-wise arithmetic of
``_scaled_mm`` itself, restated in ``scaled_mm`` below, which the gpu tests check against
``torch._scaled_mm`` on the device.

Two forms of every op:
* ``*_local``: one process holds every rank's operands in lists (collectives become cat / sum);
* ``*_dist``: runs inside a real process group (gloo) with functional collectives, used by the
  world-size-2 CPU tests and by the timed CPU baseline.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist
import torch.distributed._functional_collectives as funcol

FP8 = torch.float8_e4m3fn


# ------------------------------------------------------------------------------------------------
# scaled matmul (what aten._scaled_mm computes; call sites autoparallel/asynctp_ops.py:925-934, :1272-1281)
# ------------------------------------------------------------------------------------------------
def scaled_mm(
    A: torch.Tensor,
    B: torch.Tensor,
    A_scale: torch.Tensor,
    B_scale: torch.Tensor,
    bias: torch.Tensor | None = None,
    result_scale: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """``(A * A_scale) @ (B * B_scale) [+ bias] [* result_scale]`` rounded to ``out_dtype``.

    ``A`` [M, K] and ``B`` [K, N] are fp8 (or already-dequantised) values; ``A_scale`` is one
    value or [M, 1]; ``B_scale`` is one value or [1, N]. Scales multiply the fp32 accumulator,
    which is how row-wise scaled GEMMs apply them (dequantise after the dot product).
    """
    acc = A.to(compute_dtype) @ B.to(compute_dtype)
    acc = acc * A_scale.to(compute_dtype).reshape(-1, 1) if A_scale.numel() > 1 else acc * A_scale.to(compute_dtype)
    acc = acc * B_scale.to(compute_dtype).reshape(1, -1) if B_scale.numel() > 1 else acc * B_scale.to(compute_dtype)
    if bias is not None:
        acc = acc + bias.to(compute_dtype).reshape(1, -1)
    if result_scale is not None:
        acc = acc * result_scale.to(compute_dtype)
    return acc.to(out_dtype or A.dtype)


# ------------------------------------------------------------------------------------------------
# single-process forms
# ------------------------------------------------------------------------------------------------
def _gather_rows_front(shards: Sequence[torch.Tensor], gather_dim: int) -> torch.Tensor:
    """all_gather along dim 0 of the stacked shards, then merge the rank axis into gather_dim,
    leaving it in front (autoparallel/asynctp_ops.py:682-695: view(ws, *shape).movedim(gather_dim+1, 1).flatten(0, 1))."""
    stacked = torch.stack([s.contiguous() for s in shards])
    return stacked.movedim(gather_dim + 1, 1).flatten(0, 1)


def all_gather_matmul_local(
    A_shards: Sequence[torch.Tensor], Bs: Sequence[torch.Tensor], gather_dim: int, return_A: bool = True
) -> tuple[torch.Tensor | None, list[torch.Tensor]]:
    """autoparallel/asynctp_ops.py:672-700 (_fused_all_gather_matmul_fallback) with the ranks' shards in a list."""
    nd = A_shards[0].dim()
    if gather_dim == nd - 1:
        A = torch.cat(list(A_shards), dim=-1)                       # :686-689
        outs = [torch.matmul(A, B) for B in Bs]
        return (A if return_A else None), outs
    A = _gather_rows_front(A_shards, gather_dim)                    # :695
    outs = [torch.matmul(A, B).movedim(0, gather_dim) for B in Bs]  # :696
    return (A.movedim(0, gather_dim) if return_A else None), outs


def all_gather_scaled_matmul_local(
    A_shards: Sequence[torch.Tensor],
    Bs: Sequence[torch.Tensor],
    A_scales: Sequence[torch.Tensor],
    B_scales: Sequence[torch.Tensor],
    gather_dim: int,
    biases: Sequence[torch.Tensor | None],
    result_scales: Sequence[torch.Tensor | None],
    out_dtypes: Sequence[torch.dtype | None],
    compute_dtype: torch.dtype = torch.float32,
) -> tuple[torch.Tensor, list[torch.Tensor]]:
    """autoparallel/asynctp_ops.py:873-944. ``A_scales`` holds every rank's A_scale argument
    (identical tensors for tensor-wise / replicated scales)."""
    ws = len(A_shards)
    A = _gather_rows_front(A_shards, gather_dim)                     # :889-893
    shard, scale = A_shards[0], A_scales[0]
    if scale.shape[:-1] == shard.shape[:-1] and scale.shape[-1] == 1:        # row-wise, sharded (:377, :898-908)
        A_scale = _gather_rows_front(A_scales, gather_dim).flatten(0, -2)
    elif scale.numel() == 1:                                                  # tensor-wise (:384)
        A_scale = scale
    else:                                                                     # row-wise, replicated (:386, :909-910)
        full = list(shard.shape)
        full[gather_dim] *= ws
        if list(scale.shape[:-1]) != full[:-1]:
            raise ValueError("Invalid scale shape for fp8 all-gather")
        A_scale = scale.movedim(gather_dim, 0).flatten(0, -2)
    lead = A.shape[:-1]
    outs = []
    for B, B_scale, bias, rs, od in zip(Bs, B_scales, biases, result_scales, out_dtypes):
        C2 = scaled_mm(A.flatten(0, -2), B, A_scale, B_scale, bias, rs, od, compute_dtype)   # :925-934
        outs.append(C2.unflatten(0, lead).movedim(0, gather_dim))                               # :935-940
    return A.movedim(0, gather_dim), outs


def _reduce_scatter_local(parts: Sequence[torch.Tensor], reduce_op: str, scatter_dim: int) -> list[torch.Tensor]:
    """reduce_scatter_tensor over a list of per-rank tensors: fp32 sum (or mean) in rank order,
    rounded once to the partials' dtype, chunked along scatter_dim."""
    ws = len(parts)
    acc_dtype = torch.float64 if parts[0].dtype == torch.float64 else torch.float32
    total = parts[0].to(acc_dtype)
    for p in parts[1:]:
        total = total + p.to(acc_dtype)
    if reduce_op == "avg":
        total = total / ws
    elif reduce_op != "sum":
        raise ValueError("reduce_op must be sum or avg")
    return [c.to(parts[0].dtype).contiguous() for c in total.chunk(ws, dim=scatter_dim)]


def matmul_reduce_scatter_local(
    As: Sequence[torch.Tensor], Bs: Sequence[torch.Tensor], reduce_op: str, scatter_dim: int
) -> list[torch.Tensor]:
    """autoparallel/asynctp_ops.py:1090-1100: every rank forms ``A @ B`` in the operands' dtype
    (:1098), the results are reduce-scattered along scatter_dim. Returns one output per rank."""
    return _reduce_scatter_local([A @ B for A, B in zip(As, Bs)], reduce_op, scatter_dim)


def scaled_matmul_reduce_scatter_local(
    As: Sequence[torch.Tensor],
    Bs: Sequence[torch.Tensor],
    A_scales: Sequence[torch.Tensor],
    B_scales: Sequence[torch.Tensor],
    reduce_op: str,
    orig_scatter_dim: int,
    output_shape: Sequence[int],
    biases: Sequence[torch.Tensor | None] | None = None,
    result_scales: Sequence[torch.Tensor | None] | None = None,
    out_dtype: torch.dtype | None = None,
    compute_dtype: torch.dtype = torch.float32,
) -> list[torch.Tensor]:
    """autoparallel/asynctp_ops.py:1242-1290, one entry per rank in every list."""
    ws = len(As)
    biases = biases or [None] * ws
    result_scales = result_scales or [None] * ws
    parts = []
    for A, B, sa, sb, bias, rs in zip(As, Bs, A_scales, B_scales, biases, result_scales):
        if sa.numel() > 1:
            if sa.shape[:-1] != A.shape[:-1]:                                    # :1258-1264
                raise ValueError("For row-wise scaling, the leading dims of A_scale must match the leading dims of A")
            sa = sa.flatten(0, -2).contiguous()                                  # :1265
        C2 = scaled_mm(A.flatten(0, -2).contiguous(), B, sa, sb, bias, rs, out_dtype, compute_dtype)  # :1272-1281
        parts.append(C2.view(*output_shape[:-1], B.shape[1]))                    # :1282
    return _reduce_scatter_local(parts, reduce_op, orig_scatter_dim)             # :1283-1290


# ------------------------------------------------------------------------------------------------
# process-group forms (gloo on CPU)
# ------------------------------------------------------------------------------------------------
def _ag_front_dist(x: torch.Tensor, gather_dim: int, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    out = funcol.wait_tensor(funcol.all_gather_tensor(x.contiguous(), 0, group))
    return out.view(ws, *x.shape).movedim(gather_dim + 1, 1).flatten(0, 1)


def all_gather_matmul_dist(
    A_shard: torch.Tensor, Bs: Sequence[torch.Tensor], gather_dim: int, group=None, return_A: bool = True
) -> tuple[torch.Tensor | None, list[torch.Tensor]]:
    """autoparallel/asynctp_ops.py:672-700 over a live process group."""
    group = group or dist.group.WORLD
    ws = dist.get_world_size(group)
    if gather_dim == A_shard.dim() - 1:
        stacked = funcol.wait_tensor(funcol.all_gather_tensor(A_shard.contiguous(), 0, group))
        A = torch.cat(stacked.chunk(ws), dim=-1)
        outs = [torch.matmul(A, B) for B in Bs]
        return (A if return_A else None), outs
    A = _ag_front_dist(A_shard, gather_dim, group)
    outs = [torch.matmul(A, B).movedim(0, gather_dim) for B in Bs]
    return (A.movedim(0, gather_dim) if return_A else None), outs


def matmul_reduce_scatter_dist(
    A: torch.Tensor, B: torch.Tensor, reduce_op: str, scatter_dim: int, group=None
) -> torch.Tensor:
    """autoparallel/asynctp_ops.py:1090-1100 over a live process group."""
    group = group or dist.group.WORLD
    return funcol.wait_tensor(funcol.reduce_scatter_tensor(A @ B, reduce_op, scatter_dim, group))


def all_gather_scaled_matmul_dist(
    A_shard, Bs, A_scale, B_scales, gather_dim, biases, result_scales, out_dtypes, group=None,
    compute_dtype: torch.dtype = torch.float32,
):
    """autoparallel/asynctp_ops.py:873-944 over a live process group. fp8 payloads travel as
    bytes because gloo has no fp8 type."""
    group = group or dist.group.WORLD
    ws = dist.get_world_size(group)
    as_bytes = A_shard.view(torch.uint8) if A_shard.dtype == FP8 else A_shard
    A = _ag_front_dist(as_bytes, gather_dim, group)
    if A_shard.dtype == FP8:
        A = A.view(FP8)
    if A_scale.shape[:-1] == A_shard.shape[:-1] and A_scale.shape[-1] == 1:
        scale = _ag_front_dist(A_scale, gather_dim, group).flatten(0, -2)
    elif A_scale.numel() == 1:
        scale = A_scale
    else:
        scale = A_scale.movedim(gather_dim, 0).flatten(0, -2)
    lead = A.shape[:-1]
    outs = []
    for B, B_scale, bias, rs, od in zip(Bs, B_scales, biases, result_scales, out_dtypes):
        C2 = scaled_mm(A.flatten(0, -2), B, scale, B_scale, bias, rs, od, compute_dtype)
        outs.append(C2.unflatten(0, lead).movedim(0, gather_dim))
    return A.movedim(0, gather_dim), outs


def scaled_matmul_reduce_scatter_dist(
    A, B, A_scale, B_scale, reduce_op, orig_scatter_dim, output_shape, bias=None, result_scale=None,
    out_dtype=None, group=None, compute_dtype: torch.dtype = torch.float32,
):
    """autoparallel/asynctp_ops.py:1242-1290 over a live process group."""
    group = group or dist.group.WORLD
    if A_scale.numel() > 1:
        A_scale = A_scale.flatten(0, -2).contiguous()
    C2 = scaled_mm(A.flatten(0, -2).contiguous(), B, A_scale, B_scale, bias, result_scale, out_dtype, compute_dtype)
    C2 = C2.view(*output_shape[:-1], B.shape[1])
    return funcol.wait_tensor(funcol.reduce_scatter_tensor(C2, reduce_op, orig_scatter_dim, group))


# ------------------------------------------------------------------------------------------------
# fp64 yardstick and synthetic inputs
# ------------------------------------------------------------------------------------------------
def rel_fro_error(x: torch.Tensor, ref64: torch.Tensor) -> float:
    """``||x - ref||_F / ||ref||_F`` in fp64: the metric the tolerances are stated in."""
    d = x.detach().to("cpu", torch.float64) - ref64.to("cpu", torch.float64)
    return (d.norm() / ref64.to("cpu", torch.float64).norm().clamp_min(1e-300)).item()


def activations(rank: int, rows: int, cols: int, dtype: torch.dtype = torch.bfloat16, seed: int = 1000) -> torch.Tensor:
    """Per-rank activations ~N(0,1), seeded by rank."""
    g = torch.Generator(device="cpu").manual_seed(seed + rank)
    return torch.randn(rows, cols, generator=g, dtype=torch.float32).to(dtype)


def weights(seed: int, rows: int, cols: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> torch.Tensor:
    """Weights ~N(0, std)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(rows, cols, generator=g, dtype=torch.float32) * std).to(dtype)


def quantize_rowwise(x: torch.Tensor, dim: int) -> tuple[torch.Tensor, torch.Tensor]:
    """e4m3 row-wise quantisation: scale = amax(|x|, dim) / 448 (fp32), x8 = (x / scale).to(e4m3)."""
    x = x.to(torch.float32)
    scale = x.abs().amax(dim=dim, keepdim=True).clamp_min(1e-12) / 448.0
    return (x / scale).clamp(-448.0, 448.0).to(FP8), scale
