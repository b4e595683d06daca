"""ctypes access to the same-box GPU comparator (oracle/_ref/libqf_ref_gemv.so, built by
oracle/build_ref.py from the reference project's own kernel headers).  TEST / MEASUREMENT
INFRASTRUCTURE ONLY: used by tests/ and by bench.py's secondary `ref_gpu_kernel` figure, never by
the product."""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

from . import qf_oracle as O

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libqf_ref_gemv.so")
SHAPES = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]   # (N, K), index = the library's `shape`

_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(LIB_PATH)
        vp = ctypes.c_void_p
        L.qf_ref_gptq_gemv.restype = ctypes.c_int
        L.qf_ref_gptq_gemv.argtypes = [ctypes.c_int, ctypes.c_int, vp, vp, vp, vp, vp, vp]
        L.qf_ref_last_cuda_error.restype = ctypes.c_int
        _lib = L
    return _lib


def pack_reference_layout(q, s, z, device="cuda"):
    """Codes / scales / GPTQ zeros -> the reference's packed tensors (qfactory/convert.py:49-81 of the
    reference, restated in qf_oracle) on `device`."""
    w = torch.from_numpy(O.ref_pack_weight(q.numpy(), 4)).to(device)
    sp = torch.from_numpy(O.ref_pack_scale(s.numpy())).to(device)
    zp = torch.from_numpy(O.ref_pack_zero(z.numpy(), 4)).to(device)
    return w, sp, zp


def launch(shape: int, scheduled: int, x, w, y, s, z, stream=None) -> int:
    st = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
    return lib().qf_ref_gptq_gemv(shape, scheduled, x.data_ptr(), w.data_ptr(), y.data_ptr(), s.data_ptr(), z.data_ptr(), st)
