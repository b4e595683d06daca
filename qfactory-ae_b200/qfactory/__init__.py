"""B200-native drop-in for the quantized GEMV/GEMM path of QFactory.

`from qfactory import QLinear, QMatmul` works as with the reference package
(reference: qfactory/__init__.py:26-27); the log level still comes from
QFACTORY_LOG_LEVEL (reference: qfactory/__init__.py:5-24).
"""
import logging
import os

_level = os.environ.get("QFACTORY_LOG_LEVEL", "INFO")
assert _level in ("DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"), f"Unknown log level {_level}"
logging.getLogger(__name__).setLevel(getattr(logging, _level))

from .core import QMatmul, Matmul  # noqa: E402
from .qlinear import QLinear, GPTQLinear, GEMVLinear  # noqa: E402
from .convert import convert_params, unpack_params  # noqa: E402

__all__ = ["QLinear", "QMatmul", "Matmul", "GPTQLinear", "GEMVLinear", "convert_params", "unpack_params"]
