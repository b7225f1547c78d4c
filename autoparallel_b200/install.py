"""Installs this package's ops module under the name AutoParallel imports.

``autoparallel/asynctp.py:30`` does ``import autoparallel.asynctp_ops`` for its side effect of
registering the ``_ap_symm_mem`` ops. Calling :func:`install` before that import makes the
statement bind to :mod:`autoparallel_b200.asynctp_ops`, so the unchanged FX pass emits calls that
dispatch to the sm_100a kernels. The two modules cannot coexist in one process (an operator
namespace can be defined once), which is why this is an explicit step.
"""
from __future__ import annotations

import sys

REFERENCE_NAME = "autoparallel.asynctp_ops"


def install() -> None:
    existing = sys.modules.get(REFERENCE_NAME)
    if existing is not None and existing.__name__ != "autoparallel_b200.asynctp_ops":
        raise RuntimeError(
            f"{REFERENCE_NAME} is already imported from {getattr(existing, '__file__', '?')}; "
            "call autoparallel_b200.install.install() before importing autoparallel.asynctp"
        )
    from . import asynctp_ops

    sys.modules[REFERENCE_NAME] = asynctp_ops
    try:
        import autoparallel  # the reference package, if it is importable

        autoparallel.asynctp_ops = asynctp_ops
    except ImportError:
        pass


def retarget_symm_mem_calls(graph) -> int:
    """Point every ``torch.ops.symm_mem.fused_*`` call of an FX graph at this package's
    ``_ap_symm_mem`` op of the same name; returns how many calls were changed.

    AutoParallel's pass is a fork of ``torch._inductor.fx_passes.micro_pipeline_tp`` (header of
    autoparallel/asynctp.py) and inserts the same four calls with the same arguments, only under its
    own namespace (autoparallel/asynctp.py:653-674, :982-1010). A program that runs torch's pass
    instead of AutoParallel's can therefore use the sm_100a kernels by calling this afterwards, e.g.
    from ``torch._inductor.config.post_grad_custom_post_pass``.
    """
    import torch

    names = (
        "fused_all_gather_matmul", "fused_all_gather_scaled_matmul",
        "fused_matmul_reduce_scatter", "fused_scaled_matmul_reduce_scatter",
    )
    table = {getattr(torch.ops.symm_mem, n).default: getattr(torch.ops._ap_symm_mem, n).default for n in names}
    changed = 0
    for node in graph.nodes:
        if node.op == "call_function" and node.target in table:
            node.target = table[node.target]
            changed += 1
    return changed
