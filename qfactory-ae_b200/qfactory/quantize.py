"""fp16 weight -> group-wise asymmetric codes, the front end for "construct a layer from
an fp16 weight".  Follows the reference's test helper `asymmetric_quant`
(reference: tests/acc_gptq.py:10-29): per group of GS rows of the [K, N] weight
    scale = (max - min) / (2^b - 1)
    zero  = trunc(clamp(-min / (max - min) * (2^b - 1) - 1, min=0))      (GPTQ "zero - 1")
    code  = trunc((w - min) / (max - min) * (2^b - 1))
with all arithmetic in the weight's own dtype.  CUDA fp16 weights go through the native
`qfb_quantize` kernel (same results bit for bit, one pass over the weight); everything else
through the vectorised torch expression below.
"""
from __future__ import annotations

import torch


def asymmetric_quant(weight: torch.Tensor, group_size: int, n_bits: int):
    K, N = weight.shape
    assert K % group_size == 0
    G = K // group_size
    if weight.is_cuda and weight.dtype == torch.float16:
        from . import _native

        w = weight.contiguous()
        codes = torch.empty(K, N, dtype=torch.int32, device=w.device)
        scales = torch.empty(G, N, dtype=torch.float16, device=w.device)
        zeros = torch.empty(G, N, dtype=torch.int32, device=w.device)
        with torch.cuda.device(w.device):
            _native.check(_native.lib().qfb_quantize(w.data_ptr(), K, N, n_bits, group_size, codes.data_ptr(),
                                                     scales.data_ptr(), zeros.data_ptr(),
                                                     torch.cuda.current_stream(w.device).cuda_stream), "qfb_quantize")
        return codes, scales, zeros
    levels = 2 ** n_bits - 1
    wg = weight.reshape(G, group_size, N)
    wmax = wg.amax(dim=1)
    wmin = wg.amin(dim=1)
    span = wmax - wmin
    scales = (span / levels).to(torch.float16)
    zeros = (-wmin / span * levels - 1).clamp(min=0).to(torch.int32)
    codes = ((wg - wmin.unsqueeze(1)) / span.unsqueeze(1) * levels).to(torch.int32)
    return codes.reshape(K, N), scales, zeros
