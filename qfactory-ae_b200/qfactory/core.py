"""Operator-level API kept for drop-in compatibility with `from qfactory import QMatmul`.

In the reference `QMatmul(...).compile_profile(**flags)` enumerates a design space, JIT-
compiles each candidate and returns a closure `f(activation, weight, output, scale[, zero])`
(reference: qfactory/core/matmul.py:14-153; group-less twin `Matmul` :155-270).  Here the
closure validates the same way and calls the ahead-of-time built native kernels; the
search flags are accepted and ignored, and M may differ from the constructor's value.

The packed tensors handed to the closures are the ones `convert_params` makes; since two packed
layouts exist, the constructors take `packed_layout`: 'tile' (the default, as the default of
`convert_params` without a LAYOUT key), 'fragment' or 'auto', resolved by the same rule as
`convert_params`, and the closure passes it to the kernels.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native
from . import layout as _layout


class QMatmul:
    def __init__(self, m, n, k, nbits, sym, dtype_a=torch.float16, dtype_b=torch.int8, group_size=-1,
                 layout_="nt", base_impl=False, layout=None, packed_layout="tile"):
        lay = layout if layout is not None else layout_
        self.m, self.n, self.k = m, n, k
        self.nbits, self.sym = nbits, sym
        self.group_size = k if group_size == -1 else group_size
        assert self.k % self.group_size == 0, f"Group size {self.group_size} must divide k {self.k}"
        assert lay == "nt", f"Layout {lay} is not supported"
        assert dtype_a == torch.float16, f"Data type {dtype_a} is not supported"
        assert dtype_b == torch.int8, f"Data type {dtype_b} is not supported"
        self.packed_layout = _layout.resolve_layout(packed_layout, n, k, nbits, self.group_size, m)

    def compile_profile(self, enable_transform=False, enable_schedule=False, enable_lower=False):
        n, k, bits, gs, sym, lay = self.n, self.k, self.nbits, self.group_size, self.sym, self.packed_layout
        npad = _layout.padded_rows(n)
        L = _native.lib()
        state = {}

        def inner(activation, weight, output, scale, zero=None):
            assert activation.shape[1] == k and output.shape[1] == n
            assert activation.shape[0] == output.shape[0]
            assert weight.numel() == npad * k * bits // 8 and weight.dtype == torch.int8
            assert scale.shape == (npad, k // gs) and scale.dtype == torch.float16
            assert activation.dtype == torch.float16 and output.dtype == torch.float16
            assert activation.is_contiguous() and weight.is_contiguous() and output.is_contiguous()
            assert scale.is_contiguous()
            if not sym:
                assert zero is not None and zero.shape == (npad, k // gs) and zero.dtype == torch.int8
                assert zero.is_contiguous()
            m = activation.shape[0]
            d = _native.QfbLayer(weight.data_ptr(), scale.data_ptr(), None if sym else zero.data_ptr(), n, k, bits, gs, lay)
            key = (activation.device, m)
            if key not in state:
                nb = L.qfb_workspace_bytes(max(m, 1), n, k, bits)
                state[key] = (torch.zeros(max(nb, 16), dtype=torch.uint8, device=activation.device), nb)
            ws, nb = state[key]
            st = L.qfb_linear_forward(ctypes.byref(d), activation.data_ptr(), m, output.data_ptr(), ws.data_ptr(), nb,
                                      0, torch.cuda.current_stream(activation.device).cuda_stream)
            _native.check(st, "qfb_linear_forward")
            return st

        return inner


class Matmul:
    """Group-less twin (reference: qfactory/core/matmul.py:155-270)."""

    def __init__(self, n, k, nbits, dtype_a=torch.float16, dtype_b=torch.int8, layout_="nt", layout=None,
                 packed_layout="tile"):
        self.n, self.k, self.nbits = n, k, nbits
        lay = layout if layout is not None else layout_
        assert dtype_a == torch.float16 and dtype_b == torch.int8 and lay == "nt"
        self.packed_layout = _layout.resolve_layout(packed_layout, n, k, nbits, -1, 1)

    def compile_profile(self, enable_transform=False, enable_schedule=False, enable_lower=False):
        n, k, bits, lay = self.n, self.k, self.nbits, self.packed_layout
        npad = _layout.padded_rows(n)
        L = _native.lib()
        state = {}

        def inner(activation, weight, output):
            assert activation.shape[1] == k and output.shape[1] == n and activation.shape[0] == output.shape[0]
            assert weight.numel() == npad * k * bits // 8 and weight.dtype == torch.int8
            assert activation.dtype == torch.float16 and output.dtype == torch.float16
            assert activation.is_contiguous() and weight.is_contiguous() and output.is_contiguous()
            m = activation.shape[0]
            d = _native.QfbLayer(weight.data_ptr(), None, None, n, k, bits, -1, lay)
            key = (activation.device, m)
            if key not in state:
                nb = L.qfb_workspace_bytes(max(m, 1), n, k, bits)
                state[key] = (torch.zeros(max(nb, 16), dtype=torch.uint8, device=activation.device), nb)
            ws, nb = state[key]
            st = L.qfb_linear_forward(ctypes.byref(d), activation.data_ptr(), m, output.data_ptr(), ws.data_ptr(), nb,
                                      0, torch.cuda.current_stream(activation.device).cuda_stream)
            _native.check(st, "qfb_linear_forward")
            return st

        return inner
