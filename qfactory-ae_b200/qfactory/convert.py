"""Offline packing entry point: GPTQ-style tensors -> the B200 tile-128 layout.

Keeps the call contract of the reference's `convert_params(args, params)`
(reference: qfactory/convert.py:84-97): `args` holds K, N, NBITS and, for the grouped
path, GS; `params` is `(weight,)` for the group-less path and `(weight, scale, zero)`
otherwise, `zero=None` meaning symmetric.  Wrong arity raises ValueError, wrong
shape / dtype / value range raises AssertionError (reference: qfactory/convert.py:3-47).

What changed is the layout that comes back (see layout.py); `unpack_params` inverts it.
CUDA tensors are packed by the native `qfb_pack` kernel, CPU tensors by the torch code
in layout.py; both produce identical bytes.
"""
from __future__ import annotations

import torch

from . import layout


def _check_weight(K, N, weight, nbits):
    assert weight.shape == (K, N), f"weight must be [K={K}, N={N}]"
    assert weight.dtype == torch.int32
    lo, hi = torch.aminmax(weight)
    assert lo >= 0 and hi < 2 ** nbits, "codes out of range"


def _check_scale(K, N, GS, scale):
    assert scale.shape == (K // GS, N)
    assert scale.dtype == torch.float16


def _check_zero(K, N, GS, zero, nbits):
    assert zero.shape == (K // GS, N)
    assert zero.dtype == torch.int32
    lo, hi = torch.aminmax(zero)
    assert lo >= 0 and hi < 2 ** nbits, "zero-points out of range"


def _pack_native(K, N, nbits, GS, weight, scale, zero, lay=layout.LAYOUT_TILE):
    from . import _native

    L = _native.lib()
    dev = weight.device
    Np = layout.padded_rows(N)
    w = torch.empty(Np, K * nbits // 8, dtype=torch.int8, device=dev)
    s = z = None
    if GS != -1:
        s = torch.empty(Np, K // GS, dtype=torch.float16, device=dev)
        if zero is not None:
            z = torch.empty(Np, K // GS, dtype=torch.int8, device=dev)
    weight = weight.contiguous()
    scale_c = scale.contiguous() if scale is not None else None
    zero_c = zero.contiguous() if zero is not None else None
    with torch.cuda.device(dev):
        st = L.qfb_pack_layout(
            weight.data_ptr(),
            scale_c.data_ptr() if scale_c is not None else None,
            zero_c.data_ptr() if zero_c is not None else None,
            N, K, nbits, GS, lay,
            w.data_ptr(),
            s.data_ptr() if s is not None else None,
            z.data_ptr() if z is not None else None,
            torch.cuda.current_stream(dev).cuda_stream,
        )
    _native.check(st, "qfb_pack")
    return w, s, z


def convert_params(args, params):
    """Pack one layer.  Returns `w` (group-less) or `(w, s, z)`:
        w  int8 [Npad, K*NBITS/8]   s  fp16 [Npad, K/GS]   z  int8 [Npad, K/GS] or None
    with Npad = N rounded up to 128.  The stored zero is min(zero+1, 2^NBITS-1), as in the
    reference packer (reference: qfactory/convert.py:76).  The optional key LAYOUT ('tile', the
    default, or 'fragment') selects the packed layout (layout.py)."""
    K, N, NBITS = args["K"], args["N"], args["NBITS"]
    lay = layout.resolve_layout(args.get("LAYOUT", "tile"), N, K, NBITS, args.get("GS", -1))
    frag = lay == layout.LAYOUT_FRAGMENT
    if "GS" not in args:
        if len(params) != 1:
            raise ValueError("gemv requires 1 parameters")
        (weight,) = params
        layout.check_shape(N, K, NBITS, -1)
        _check_weight(K, N, weight, NBITS)
        if weight.is_cuda:
            return _pack_native(K, N, NBITS, -1, weight, None, None, lay)[0]
        return layout.pack_weight_fragment(weight, NBITS) if frag else layout.pack_weight(weight, NBITS)
    if len(params) != 3:
        raise ValueError("gptq_gemv requires 3 parameters")
    weight, scale, zero = params
    GS = args["GS"]
    layout.check_shape(N, K, NBITS, GS)
    _check_weight(K, N, weight, NBITS)
    _check_scale(K, N, GS, scale)
    if zero is not None:
        _check_zero(K, N, GS, zero, NBITS)
    if weight.is_cuda:
        return _pack_native(K, N, NBITS, GS, weight, scale, zero, lay)
    if frag:
        return (layout.pack_weight_fragment(weight, NBITS), layout.pack_scale_fragment(scale),
                layout.pack_zero_fragment(zero, NBITS) if zero is not None else None)
    w = layout.pack_weight(weight, NBITS)
    s = layout.pack_scale(scale)
    z = layout.pack_zero(zero, NBITS) if zero is not None else None
    return w, s, z


def unpack_params(args, packed):
    """Inverse of convert_params: returns codes int32 [K,N] (group-less) or
    (codes, scales fp16 [K/GS,N], effective zeros int32 [K/GS,N] or None)."""
    K, N, NBITS = args["K"], args["N"], args["NBITS"]
    frag = layout.resolve_layout(args.get("LAYOUT", "tile"), N, K, NBITS, args.get("GS", -1)) == layout.LAYOUT_FRAGMENT
    if "GS" not in args:
        w = packed[0] if isinstance(packed, (tuple, list)) else packed
        return layout.unpack_weight_fragment(w, N, K, NBITS) if frag else layout.unpack_weight(w, N, K, NBITS)
    w, s, z = packed
    if frag:
        return (layout.unpack_weight_fragment(w, N, K, NBITS), layout.unpack_scale_fragment(s, N),
                layout.unpack_zero_fragment(z, N) if z is not None else None)
    return (
        layout.unpack_weight(w, N, K, NBITS),
        layout.unpack_scale(s, N),
        layout.unpack_zero(z, N) if z is not None else None,
    )
