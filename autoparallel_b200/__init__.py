"""B200-native async tensor-parallel ops: a drop-in for AutoParallel's ``autoparallel.asynctp_ops``."""

__all__ = ["__version__"]
__version__ = "0.1.0"
