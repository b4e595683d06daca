"""ctypes binding of the native library (lib/libqfactory_b200.so, C ABI in
include/qfactory_b200.h).

The reference binds its JIT-built kernels the same way: `ctypes.CDLL(...).launch` with
`c_void_p` tensor pointers (reference: qfactory/jit/runtime.py:22-49).  There is no
Python or CPU fallback: if the library is missing, `lib()` raises.
"""
from __future__ import annotations

import ctypes
import os

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_ROOT, "lib", "libqfactory_b200.so")

QFB_OK = 0
FLAG_PDL = 1
FLAG_FORCE_SIMT = 2
FLAG_FORCE_TENSOR = 4
FLAG_NO_SYNC = 8
FLAG_TEST_STALLED_WAIT = 16

EXPORTS = (
    "qfb_version", "qfb_status_string", "qfb_last_cuda_error",
    "qfb_packed_weight_bytes", "qfb_packed_scale_bytes", "qfb_packed_zero_bytes",
    "qfb_workspace_bytes", "qfb_workspace_init",
    "qfb_linear_forward", "qfb_linear_forward_host", "qfb_linear_silu_mul_forward", "qfb_select_kernel",
    "qfb_set_gemv_tuning", "qfb_get_last_launch", "qfb_set_tensor_min_batch", "qfb_set_tensor_split", "qfb_set_tensor_decode_groups", "qfb_set_tensor_batch_tile", "qfb_set_cluster_reduce", "qfb_read_status",
    "qfb_pack", "qfb_pack_layout", "qfb_layout_supported", "qfb_unpack_codes", "qfb_dequantize",
    "qfb_gemv_forward_static", "qfb_static_scratch_capacity",
    "qfb_rmsnorm", "qfb_add_rmsnorm", "qfb_silu_mul", "qfb_rope_cache", "qfb_quantize", "qfb_decode_attention", "qfb_decode_attention_rope",
    "qfb_comm_buffer_bytes", "qfb_comm_max_rows", "qfb_comm_alloc", "qfb_comm_free", "qfb_comm_open", "qfb_comm_close",
    "qfb_comm_create", "qfb_comm_destroy", "qfb_comm_set_timeout_us", "qfb_comm_slot", "qfb_comm_region", "qfb_comm_epoch",
    "qfb_allreduce_add_rmsnorm", "qfb_allreduce_add_rmsnorm_pushed", "qfb_linear_forward_reduce", "qfb_linear_addnorm_forward", "qfb_comm_step_begin", "qfb_linear_forward_reduce_step",
    "qfb_linear_silu_mul_forward_reduce_step", "qfb_linear_collect_addnorm_forward", "qfb_allreduce_add_rmsnorm_step",
    "qfb_linear_addnorm_supported",
    "qfb_linear_silu_mul_forward_reduce", "qfb_comm_read_status", "qfb_comm_last_cuda_error",
)


class QfbLayer(ctypes.Structure):
    """Mirror of `struct qfb_layer`."""

    _fields_ = [
        ("qweight", ctypes.c_void_p),
        ("scales", ctypes.c_void_p),
        ("zeros", ctypes.c_void_p),
        ("n", ctypes.c_int32),
        ("k", ctypes.c_int32),
        ("bits", ctypes.c_int32),
        ("group_size", ctypes.c_int32),
        ("layout", ctypes.c_int32),
    ]


class NativeError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    """Load the native library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeError(
            f"native library {LIB_PATH} not found: build it with "
            f"`python {os.path.join(_PKG_ROOT, 'build.py')}` (needs nvcc); there is no fallback path"
        )
    L = ctypes.CDLL(LIB_PATH)
    vp, i32, u32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    LP = ctypes.POINTER(QfbLayer)
    L.qfb_version.restype = i32
    L.qfb_status_string.restype = ctypes.c_char_p
    L.qfb_status_string.argtypes = [i32]
    L.qfb_last_cuda_error.restype = i32
    for f in (L.qfb_packed_weight_bytes, L.qfb_packed_scale_bytes, L.qfb_packed_zero_bytes):
        f.restype = sz
        f.argtypes = [i32, i32, i32]
    L.qfb_workspace_bytes.restype = sz
    L.qfb_workspace_bytes.argtypes = [i32, i32, i32, i32]
    L.qfb_workspace_init.restype = i32
    L.qfb_workspace_init.argtypes = [vp, sz, vp]
    L.qfb_linear_forward.restype = i32
    L.qfb_linear_forward.argtypes = [LP, vp, i32, vp, vp, sz, u32, vp]
    L.qfb_linear_silu_mul_forward.restype = i32
    L.qfb_linear_silu_mul_forward.argtypes = [LP, vp, i32, vp, vp, sz, u32, vp]
    L.qfb_linear_forward_host.restype = i32
    L.qfb_linear_forward_host.argtypes = [LP, vp, i32, vp, vp, vp, vp, sz, u32, vp]
    L.qfb_select_kernel.restype = i32
    L.qfb_select_kernel.argtypes = [i32, i32, i32, i32, u32]
    L.qfb_set_gemv_tuning.restype = None
    L.qfb_set_gemv_tuning.argtypes = [i32, i32]
    L.qfb_set_tensor_min_batch.restype = None
    L.qfb_set_tensor_min_batch.argtypes = [i32]
    L.qfb_set_tensor_split.restype = None
    L.qfb_set_tensor_split.argtypes = [i32]
    L.qfb_set_tensor_decode_groups.restype = None
    L.qfb_set_tensor_decode_groups.argtypes = [i32]
    L.qfb_set_tensor_batch_tile.restype = None
    L.qfb_set_tensor_batch_tile.argtypes = [i32]
    L.qfb_set_cluster_reduce.restype = None
    L.qfb_set_cluster_reduce.argtypes = [i32]
    L.qfb_read_status.restype = i32
    L.qfb_read_status.argtypes = [vp, vp, ctypes.POINTER(u32)]
    L.qfb_get_last_launch.restype = None
    L.qfb_get_last_launch.argtypes = [ctypes.POINTER(i32)] * 5
    L.qfb_pack.restype = i32
    L.qfb_pack.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.qfb_pack_layout.restype = i32
    L.qfb_pack_layout.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp]
    L.qfb_layout_supported.restype = i32
    L.qfb_layout_supported.argtypes = [i32, i32, i32, i32, i32]
    L.qfb_unpack_codes.restype = i32
    L.qfb_unpack_codes.argtypes = [LP, vp, vp]
    L.qfb_dequantize.restype = i32
    L.qfb_dequantize.argtypes = [LP, vp, vp]
    L.qfb_gemv_forward_static.restype = i32
    L.qfb_gemv_forward_static.argtypes = [LP, vp, i32, vp, u32, vp]
    L.qfb_static_scratch_capacity.restype = sz
    L.qfb_rmsnorm.restype = i32
    L.qfb_rmsnorm.argtypes = [vp, vp, vp, i32, i32, ctypes.c_float, vp]
    L.qfb_add_rmsnorm.restype = i32
    L.qfb_add_rmsnorm.argtypes = [vp, vp, vp, vp, i32, i32, ctypes.c_float, vp]
    L.qfb_rope_cache.restype = i32
    L.qfb_rope_cache.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
    L.qfb_decode_attention.restype = i32
    L.qfb_decode_attention.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    L.qfb_decode_attention_rope.restype = i32
    L.qfb_decode_attention_rope.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    L.qfb_quantize.restype = i32
    L.qfb_quantize.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.qfb_silu_mul.restype = i32
    L.qfb_silu_mul.argtypes = [vp, vp, i32, i32, vp]
    L.qfb_comm_buffer_bytes.restype = sz
    L.qfb_comm_buffer_bytes.argtypes = [sz]
    L.qfb_comm_max_rows.restype = i32
    L.qfb_comm_alloc.restype = i32
    L.qfb_comm_alloc.argtypes = [sz, ctypes.POINTER(vp), vp]
    L.qfb_comm_free.restype = i32
    L.qfb_comm_free.argtypes = [vp]
    L.qfb_comm_open.restype = i32
    L.qfb_comm_open.argtypes = [vp, ctypes.POINTER(vp)]
    L.qfb_comm_close.restype = i32
    L.qfb_comm_close.argtypes = [vp]
    L.qfb_comm_create.restype = i32
    L.qfb_comm_create.argtypes = [i32, i32, ctypes.POINTER(vp), sz, ctypes.POINTER(vp)]
    L.qfb_comm_destroy.restype = None
    L.qfb_comm_destroy.argtypes = [vp]
    L.qfb_comm_set_timeout_us.restype = None
    L.qfb_comm_set_timeout_us.argtypes = [vp, u32]
    L.qfb_comm_slot.restype = vp
    L.qfb_comm_slot.argtypes = [vp, i32]
    L.qfb_comm_region.restype = vp
    L.qfb_comm_region.argtypes = [vp, i32, i32]
    L.qfb_comm_epoch.restype = i32
    L.qfb_comm_epoch.argtypes = [vp, i32, vp, ctypes.POINTER(u32)]
    L.qfb_allreduce_add_rmsnorm.restype = i32
    L.qfb_allreduce_add_rmsnorm.argtypes = [vp, i32, vp, vp, vp, i32, i32, ctypes.c_float, vp]
    L.qfb_allreduce_add_rmsnorm_pushed.restype = i32
    L.qfb_allreduce_add_rmsnorm_pushed.argtypes = [vp, i32, vp, vp, vp, i32, i32, ctypes.c_float, vp]
    L.qfb_comm_step_begin.restype = i32
    L.qfb_comm_step_begin.argtypes = [vp, vp]
    L.qfb_linear_forward_reduce_step.restype = i32
    L.qfb_linear_forward_reduce_step.argtypes = [LP, vp, i32, vp, i32, i32, vp, sz, u32, vp]
    L.qfb_linear_silu_mul_forward_reduce_step.restype = i32
    L.qfb_linear_silu_mul_forward_reduce_step.argtypes = [LP, vp, i32, vp, i32, i32, vp, sz, u32, vp]
    L.qfb_linear_collect_addnorm_forward.restype = i32
    L.qfb_linear_collect_addnorm_forward.argtypes = [LP, vp, i32, i32, vp, vp, vp, ctypes.c_float, i32, vp, vp, sz, u32, vp]
    L.qfb_allreduce_add_rmsnorm_step.restype = i32
    L.qfb_allreduce_add_rmsnorm_step.argtypes = [vp, i32, i32, vp, vp, vp, i32, i32, ctypes.c_float, vp]
    L.qfb_linear_addnorm_supported.restype = i32
    L.qfb_linear_addnorm_supported.argtypes = [LP, i32]
    L.qfb_linear_addnorm_forward.restype = i32
    L.qfb_linear_addnorm_forward.argtypes = [LP, vp, vp, vp, vp, ctypes.c_float, i32, vp, vp, sz, u32, vp]
    L.qfb_linear_forward_reduce.restype = i32
    L.qfb_linear_forward_reduce.argtypes = [LP, vp, i32, vp, i32, vp, sz, u32, vp]
    L.qfb_linear_silu_mul_forward_reduce.restype = i32
    L.qfb_linear_silu_mul_forward_reduce.argtypes = [LP, vp, i32, vp, i32, vp, sz, u32, vp]
    L.qfb_comm_read_status.restype = i32
    L.qfb_comm_read_status.argtypes = [vp, vp, ctypes.POINTER(u32)]
    L.qfb_comm_last_cuda_error.restype = i32
    _lib = L
    return L


def check(status: int, what: str = "qfactory_b200") -> None:
    if status != QFB_OK:
        L = lib()
        msg = L.qfb_status_string(status).decode()
        extra = f" (cudaError {L.qfb_last_cuda_error()})" if status == 6 else ""
        raise NativeError(f"{what}: {msg}{extra}")


def last_launch() -> dict:
    v = [ctypes.c_int(0) for _ in range(5)]
    lib().qfb_get_last_launch(*[ctypes.byref(x) for x in v])
    return dict(zip(("kernel", "grid_x", "grid_y", "block", "smem"), (x.value for x in v)))


def version_or_zero() -> int:
    """`qfb_version()` of the built library, 0 when it has not been built (state_dict tags only)."""
    try:
        return int(lib().qfb_version())
    except NativeError:
        return 0
