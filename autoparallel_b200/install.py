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
