"""GPTQ checkpoint tensors -> the tensors `QLinear.init` takes.

A GPTQ checkpoint stores, per linear layer (the parameters the reference's vLLM hook registers,
reference: third_party/vllm-qfactory.patch:123-186):

    qweight  int32 [K / pf, N]     pf = 32 / bits codes per word, packed along K, code k of a
                                   word at bits [(k % pf) * bits, +bits)
    qzeros   int32 [K / GS, N / pf] zero-points packed along N the same way, stored MINUS ONE
                                   (the "zero - 1" convention the reference's packer undoes with
                                   its +1, reference: qfactory/convert.py:76)
    scales   fp16  [K / GS, N]
    g_idx    int32 [K]             group of every input feature; k // GS without act-order

The reference hook never unpacked these (weight loading is commented out there,
reference: third_party/vllm-qfactory.patch:223-228); this module does, in vectorised torch on
whatever device the tensors live on.
"""
from __future__ import annotations

import torch


def unpack_qweight(qweight: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 [K/pf, N] -> int32 codes [K, N]."""
    assert bits in (2, 4, 8), "GPTQ int32 packing covers 2/4/8 bits"
    pf = 32 // bits
    Kp, N = qweight.shape
    sh = (torch.arange(pf, device=qweight.device, dtype=torch.int32) * bits).view(1, pf, 1)
    q = (qweight.view(Kp, 1, N) >> sh) & ((1 << bits) - 1)
    return q.reshape(Kp * pf, N).to(torch.int32)


def unpack_qzeros(qzeros: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 [G, N/pf] -> int32 stored zeros [G, N] (still "zero - 1": pass them on as they are)."""
    assert bits in (2, 4, 8)
    pf = 32 // bits
    G, Np = qzeros.shape
    sh = (torch.arange(pf, device=qzeros.device, dtype=torch.int32) * bits).view(1, 1, pf)
    z = (qzeros.view(G, Np, 1) >> sh) & ((1 << bits) - 1)
    return z.reshape(G, Np * pf).to(torch.int32)


def pack_qweight(q: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of unpack_qweight (used by tests and to fabricate checkpoints)."""
    pf = 32 // bits
    K, N = q.shape
    sh = (torch.arange(pf, device=q.device, dtype=torch.int64) * bits).view(1, pf, 1)
    w = (q.view(K // pf, pf, N).to(torch.int64) << sh).sum(1)
    return w.where(w < 2**31, w - 2**32).to(torch.int32)


def pack_qzeros(z: torch.Tensor, bits: int) -> torch.Tensor:
    pf = 32 // bits
    G, N = z.shape
    sh = (torch.arange(pf, device=z.device, dtype=torch.int64) * bits).view(1, 1, pf)
    w = (z.view(G, N // pf, pf).to(torch.int64) << sh).sum(2)
    return w.where(w < 2**31, w - 2**32).to(torch.int32)


def check_g_idx(g_idx: torch.Tensor, group_size: int) -> bool:
    """True when g_idx is the trivial k // group_size map (no activation reordering)."""
    K = g_idx.numel()
    return bool(torch.equal(g_idx.to(torch.int64).cpu(), torch.arange(K) // group_size))


def layer_from_gptq(qweight, qzeros, scales, bits: int, group_size: int, g_idx=None, sym: bool = False,
                    batch_size: int = 1):
    """Build a packed QLinear layer from GPTQ checkpoint tensors."""
    from .qlinear import QLinear

    if g_idx is not None and not check_g_idx(g_idx, group_size):
        raise ValueError("activation-reordered GPTQ checkpoints (desc_act=True) are not supported")
    q = unpack_qweight(qweight, bits)
    K, N = q.shape
    z = None if sym else unpack_qzeros(qzeros, bits)[:, :N].contiguous()
    return QLinear.init(batch_size, K, N, bits, q, group_size, scales.to(torch.float16).contiguous(), z)
