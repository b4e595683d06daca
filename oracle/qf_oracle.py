"""CPU oracle for the weight-only-quantized linear path  y = x . dequant(W)^T.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is
the checker used by tests/, by the smoke entry and by the CPU-baseline / reference
arms of bench.py.  The product path runs hand-written CUDA and raises when the
native library is missing.

Every function restates, in numpy / torch-on-CPU, one piece of the reference
project's own algorithm and cites the reference file:line it follows (paths are
relative to the reference project's root):

  * the reference packed layout           qfactory/convert.py:49-97
  * the kernel-side decode semantics      qfactory/include/utils.h:46-62,
                                          qfactory/include/gptq_gemv.h:65-90
  * the dequantize-then-matmul test path  tests/acc_gptq.py:10-38,52
  * the group-less path                   tests/acc_gemv.py:12-14

Parity pin: the reference ships no golden vectors.  tests/golden/ holds small
fixtures produced by importing the reference's own Python (convert_params,
asymmetric_quant, dequant) with the generating script beside them; the test-suite
checks every function here against those fixtures.  The 3-bit width has no
reference packing or kernel at all: for 3-bit only the generic dequant formula is
pinned ("parity unpinned" at the packing level).

Zero-point convention (this matters, the reference is not self-consistent):
the reference API takes GPTQ-style zeros `z`; its packer stores
`z_eff = min(z + 1, 2^b - 1)` (qfactory/convert.py:76) and its kernel computes
`(q - z_eff) * s` (qfactory/include/utils.h:53-60).  Its test helper computes
`(q - (z + 1)) * s` without the clamp (tests/acc_gptq.py:36).  The two agree unless
`z == 2^b - 1`.  The oracle for kernel parity is `dequant_effective`, i.e. the
packer + kernel semantics; `dequant_unclamped` restates the test helper.
"""
from __future__ import annotations

import time

import numpy as np
import torch

# --------------------------------------------------------------------------
# Reference packed layout (qfactory/convert.py)
# --------------------------------------------------------------------------


def ref_permute_order(bits: int) -> list[int]:
    """Field order inside one little-endian u32 (qfactory/convert.py:49-53).

    Field j (bits [j*b, (j+1)*b)) of the word holds element order[j] of the run of
    32/b consecutive k.  For 2/4-bit the even elements fill the low 16 bits and the
    odd ones the high 16 bits; 8-bit is the identity.  3-bit is absent upstream.
    """
    if bits == 8:
        return [0, 1, 2, 3]
    if bits in (2, 4):
        pf = 32 // bits
        return list(range(0, pf, 2)) + list(range(1, pf, 2))
    raise KeyError(bits)


def ref_pack_weight(q: np.ndarray, bits: int) -> np.ndarray:
    """int32 codes [K, N] -> int8 [N, K*bits/8]  (qfactory/convert.py:55-68)."""
    K, N = q.shape
    pf = 32 // bits
    assert K % pf == 0
    order = ref_permute_order(bits)
    words = np.zeros((K // pf, N), dtype=np.uint32)
    qv = q.astype(np.uint32).reshape(K // pf, pf, N)
    for j in range(pf):
        words |= qv[:, order[j], :] << np.uint32(j * bits)
    # each word is emitted as 4 little-endian bytes along K, then transposed N-major
    by = np.stack([(words >> np.uint32(8 * i)) & np.uint32(0xFF) for i in range(4)], axis=1)
    by = by.reshape(K // pf * 4, N).astype(np.uint8)
    return np.ascontiguousarray(by.T).view(np.int8)


def ref_unpack_weight(w: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of ref_pack_weight: int8 [N, K*bits/8] -> int32 codes [K, N]."""
    N, nb = w.shape
    pf = 32 // bits
    words = np.ascontiguousarray(w).view(np.uint8).reshape(N, nb // 4, 4).astype(np.uint32)
    words = words[:, :, 0] | (words[:, :, 1] << 8) | (words[:, :, 2] << 16) | (words[:, :, 3] << 24)
    order = ref_permute_order(bits)
    out = np.zeros((N, nb // 4, pf), dtype=np.int32)
    mask = np.uint32((1 << bits) - 1)
    for j in range(pf):
        out[:, :, order[j]] = ((words >> np.uint32(j * bits)) & mask).astype(np.int32)
    return np.ascontiguousarray(out.reshape(N, -1).T)


def effective_zero(z: np.ndarray, bits: int) -> np.ndarray:
    """z_eff = min(z + 1, 2^b - 1)  (qfactory/convert.py:76)."""
    return np.minimum(z.astype(np.int64) + 1, (1 << bits) - 1).astype(np.int32)


def symmetric_zero(bits: int) -> int:
    """Symmetric layers subtract 2^(b-1) with no +1 (qfactory/include/gptq_gemv.h:72-73)."""
    return 1 << (bits - 1)


def ref_pack_zero(z: np.ndarray, bits: int) -> np.ndarray:
    """int32 zeros [G, N] -> int8 [N, G/(8/b)] holding z_eff (qfactory/convert.py:74-81)."""
    G, N = z.shape
    pf8 = 8 // bits
    assert G % pf8 == 0
    ze = effective_zero(z, bits).astype(np.uint8).reshape(G // pf8, pf8, N)
    out = np.zeros((G // pf8, N), dtype=np.uint8)
    for i in range(pf8):
        out |= (ze[:, i, :] << np.uint8(i * bits)).astype(np.uint8)
    return np.ascontiguousarray(out.T).view(np.int8)


def ref_unpack_zero(zp: np.ndarray, bits: int) -> np.ndarray:
    """int8 [N, G/(8/b)] -> effective zeros int32 [G, N]; the read-back of
    qfactory/include/gptq_gemv.h:76-80 (byte >> ((g % pf8) * b)) & mask."""
    N, nb = zp.shape
    pf8 = 8 // bits
    b = np.ascontiguousarray(zp).view(np.uint8)
    out = np.zeros((N, nb, pf8), dtype=np.int32)
    for i in range(pf8):
        out[:, :, i] = (b >> np.uint8(i * bits)) & np.uint8((1 << bits) - 1)
    return np.ascontiguousarray(out.reshape(N, -1).T)


def ref_pack_scale(s: np.ndarray) -> np.ndarray:
    """fp16 [G, N] -> fp16 [N, G]  (qfactory/convert.py:70-72)."""
    return np.ascontiguousarray(s.T)


def ref_convert_params(args: dict, params: tuple):
    """Dispatch of qfactory/convert.py:84-97 on numpy arrays."""
    K, N, bits = args["K"], args["N"], args["NBITS"]
    if "GS" not in args:
        if len(params) != 1:
            raise ValueError("gemv requires 1 parameters")
        (q,) = params
        assert q.shape == (K, N) and q.min() >= 0 and q.max() < (1 << bits)
        return ref_pack_weight(q, bits)
    if len(params) != 3:
        raise ValueError("gptq_gemv requires 3 parameters")
    q, s, z = params
    GS = args["GS"]
    assert q.shape == (K, N) and q.min() >= 0 and q.max() < (1 << bits)
    assert s.shape == (K // GS, N) and s.dtype == np.float16
    w = ref_pack_weight(q, bits)
    sp = ref_pack_scale(s)
    zp = None
    if z is not None:
        assert z.shape == (K // GS, N) and z.min() >= 0 and z.max() < (1 << bits)
        zp = ref_pack_zero(z, bits)
    return w, sp, zp


# --------------------------------------------------------------------------
# Dequantize-then-matmul (tests/acc_gptq.py, tests/acc_gemv.py)
# --------------------------------------------------------------------------


def _t(a, dtype=None):
    t = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))
    return t if dtype is None else t.to(dtype)


def dequant_unclamped(q, s, z) -> torch.Tensor:
    """(q - (z[k//GS] + 1)) * s[k//GS] -> fp16 [K, N]  (tests/acc_gptq.py:31-38)."""
    q, s, z = _t(q, torch.int32), _t(s, torch.float16), _t(z, torch.int32)
    K = q.shape[0]
    GS = K // s.shape[0]
    kidx = torch.arange(K) // GS
    return (q - (z[kidx] + 1)) * s[kidx]


def dequant_effective(q, s, z_eff) -> torch.Tensor:
    """(q - z_eff[k//GS]) * s[k//GS] -> fp16 [K, N]: the packer + kernel semantics
    (qfactory/convert.py:76 with qfactory/include/utils.h:53-60).  `z_eff` may be an
    int for the symmetric case.  q - z_eff is exact in fp16; the product rounds once,
    exactly as fma.rn.f16x2 with a zero addend does in the reference kernel."""
    q, s = _t(q, torch.int32), _t(s, torch.float16)
    K = q.shape[0]
    GS = K // s.shape[0]
    kidx = torch.arange(K) // GS
    if isinstance(z_eff, (int, np.integer)):
        d = q - int(z_eff)
    else:
        d = q - _t(z_eff, torch.int32)[kidx]
    return d * s[kidx]


def qlinear_fp16(x, wdq: torch.Tensor) -> torch.Tensor:
    """x[M,K] fp16 @ dequantised fp16 weight [K,N] -> fp16  (tests/acc_gptq.py:52)."""
    return _t(x, torch.float16) @ wdq


def qlinear_exact(x, wdq: torch.Tensor) -> np.ndarray:
    """Same contraction in float64 over the fp16-rounded operands: the value both the
    fp16 CPU matmul and an fp32-accumulating kernel approximate."""
    return _t(x, torch.float16).double().numpy() @ wdq.double().numpy()


def gemv_groupless_fp16(x, q) -> torch.Tensor:
    """x @ codes.half(): raw unsigned codes, no scale or zero (tests/acc_gemv.py:14)."""
    return _t(x, torch.float16) @ _t(q, torch.int32).to(torch.float16)


def gemv_groupless_exact(x, q) -> np.ndarray:
    return _t(x, torch.float16).double().numpy() @ _t(q, torch.int32).double().numpy()


def asymmetric_quant(weight, GS: int, bits: int):
    """fp16 weight [K,N] -> (codes i32 [K,N], scales f16 [K/GS,N], zeros i32 [K/GS,N])
    following tests/acc_gptq.py:10-29: per group, scale = (max-min)/(2^b-1),
    zero = clamp(-min/(max-min)*(2^b-1) - 1, 0) truncated, code = trunc((w-min)/(max-min)*(2^b-1)).
    All arithmetic stays in the weight's dtype, as upstream."""
    w = _t(weight)
    K, N = w.shape
    assert K % GS == 0
    G = K // GS
    qr = (1 << bits) - 1
    wg = w.reshape(G, GS, N)
    wmax = wg.max(dim=1).values
    wmin = wg.min(dim=1).values
    scales = ((wmax - wmin) / qr).to(torch.float16)
    zeros = (-wmin / (wmax - wmin) * qr - 1).clamp(min=0).to(torch.int32)
    q = ((wg - wmin[:, None, :]) / (wmax - wmin)[:, None, :] * qr).to(torch.int32)
    return q.reshape(K, N), scales, zeros


# --------------------------------------------------------------------------
# Seeded synthetic inputs with the benchmark configurations' distributions
# --------------------------------------------------------------------------


def make_case(M: int, N: int, K: int, bits: int, GS: int, sym: bool = False, seed: int = 0):
    """x ~ N(0,1) fp16 [M,K]; codes uniform in [0, 2^b); scales ~ U(0.002, 0.02) fp16
    [K/GS, N]; zeros uniform in [0, 2^b) (API / GPTQ convention) or None when sym.
    GS == -1 gives the group-less case (codes only)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.float16)
    q = torch.randint(0, 1 << bits, (K, N), generator=g, dtype=torch.int32)
    if GS == -1:
        return x, q, None, None
    s = (torch.rand(K // GS, N, generator=g) * 0.018 + 0.002).to(torch.float16)
    z = None if sym else torch.randint(0, 1 << bits, (K // GS, N), generator=g, dtype=torch.int32)
    return x, q, s, z


def reference_forward(x, q, s, z, bits: int):
    """Oracle output (fp16 tensor, float64 array) for one layer with API-convention
    zeros `z` (None = symmetric, s None = group-less)."""
    if s is None:
        return gemv_groupless_fp16(x, q), gemv_groupless_exact(x, q)
    ze = symmetric_zero(bits) if z is None else effective_zero(_t(z).numpy(), bits)
    wdq = dequant_effective(q, s, ze)
    return qlinear_fp16(x, wdq), qlinear_exact(x, wdq)


def algorithmic_bytes(M, N, K, bits, GS, sym) -> int:
    """The reference's own footprint model (reproduce/fig9/plot_bandwidth_size.py:37-44):
    activations + outputs + packed codes + fp16 scales + packed zeros (asym only)."""
    b = 2 * (M * K + M * N) + N * K * bits // 8
    if GS != -1:
        b += (K // GS) * N * 2
        if not sym:
            b += (K // GS) * N * bits // 8
    return b


def time_cpu_path(x, q, s, z, bits: int, repeats: int = 3):
    """Wall time of the reference's CPU path, dequant (tests/acc_gptq.py:31-38) then fp16
    matmul (:52), on torch CPU tensors with torch's current thread count.  Returns
    (best_seconds, threads)."""
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        if s is None:
            gemv_groupless_fp16(x, q)
        else:
            ze = symmetric_zero(bits) if z is None else effective_zero(_t(z).numpy(), bits)
            qlinear_fp16(x, dequant_effective(q, s, ze))
        best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads()
