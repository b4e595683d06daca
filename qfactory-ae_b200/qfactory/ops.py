"""Element-wise neighbours of the quantized linears in a decoder layer, one native launch each
(C ABI: qfb_rmsnorm, qfb_silu_mul, qfb_rope_cache in include/qfactory_b200.h).  The reference
leaves these to its serving stack (reference:
third_party/vllm-bitblas/vllm/model_executor/models/llama.py:60-120, 260-285); here they keep a
decode step from being dominated by chains of small framework kernels between the linears.
CUDA fp16 tensors only; there is no CPU path."""
from __future__ import annotations

import torch

from . import _native


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp16(x * rsqrt(mean(x^2, -1) + eps)) * weight over the last dimension."""
    assert x.is_cuda and x.dtype == torch.float16 and x.is_contiguous() and weight.dtype == torch.float16
    d = x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    _native.check(_native.lib().qfb_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.numel() // d, d, eps,
                                            _stream(x)), "qfb_rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """x += residual (in place, fp16), then the RMS norm of the sum: returns the normed tensor."""
    assert x.is_cuda and x.dtype == torch.float16 and x.is_contiguous()
    assert residual.shape == x.shape and residual.dtype == torch.float16 and residual.is_contiguous()
    d = x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    _native.check(_native.lib().qfb_add_rmsnorm(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                                x.numel() // d, d, eps, _stream(x)), "qfb_add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """silu(gate_up[..., :h]) * gate_up[..., h:] with h = half of the last dimension."""
    assert gate_up.is_cuda and gate_up.dtype == torch.float16 and gate_up.is_contiguous()
    half = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * half)
    if out is None:
        out = torch.empty(*gate_up.shape[:-1], half, dtype=torch.float16, device=gate_up.device)
    _native.check(_native.lib().qfb_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, half, _stream(gate_up)),
                  "qfb_silu_mul")
    return out


def rope_cache(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor,
               v_cache: torch.Tensor, q_heads: int, kv_heads: int) -> None:
    """In-place rotary embedding of the query and key heads of qkv [B, T, q_heads + 2 kv_heads, hd]
    at positions pos [T] (int64), and the write of the rotated keys and the values into the caches
    [B, kv_heads, max_len, hd]."""
    B, T, H, hd = qkv.shape
    assert H == q_heads + 2 * kv_heads and qkv.is_contiguous() and qkv.dtype == torch.float16
    assert pos.dtype == torch.int64 and pos.numel() == T and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape == v_cache.shape == (B, kv_heads, k_cache.shape[2], hd)
    _native.check(_native.lib().qfb_rope_cache(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(),
                                               k_cache.data_ptr(), v_cache.data_ptr(), B, T, q_heads, kv_heads, hd,
                                               k_cache.shape[2], _stream(qkv)), "qfb_rope_cache")


def decode_attention_supported(q_heads: int, kv_heads: int, head_dim: int, max_len: int) -> bool:
    """Shapes `decode_attention` serves (the decoder falls back to the framework's attention otherwise)."""
    return (head_dim == 128 and kv_heads > 0 and q_heads % kv_heads == 0 and q_heads // kv_heads in (1, 2, 4, 8)
            and 0 < max_len <= 16384)


def decode_attention(qkv: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, q_heads: int,
                     kv_heads: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of ONE new token per batch row over the static cache: qkv [B, 1, q_heads + 2 kv_heads, hd]
    with the queries already rotated (`rope_cache`, which also wrote position pos into the caches),
    pos [1] int64 on the device, caches [B, kv_heads, max_len, hd].  Returns [B, q_heads * hd], the
    O projection's input."""
    B, T, H, hd = qkv.shape
    assert T == 1 and H == q_heads + 2 * kv_heads and qkv.is_contiguous() and qkv.dtype == torch.float16
    assert pos.dtype == torch.int64 and pos.numel() == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape == v_cache.shape == (B, kv_heads, k_cache.shape[2], hd)
    if out is None:
        out = torch.empty(B, q_heads * hd, dtype=torch.float16, device=qkv.device)
    _native.check(_native.lib().qfb_decode_attention(qkv.data_ptr(), pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                     out.data_ptr(), B, q_heads, kv_heads, hd, k_cache.shape[2],
                                                     _stream(qkv)), "qfb_decode_attention")
    return out


def decode_attention_rope(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor,
                          v_cache: torch.Tensor, q_heads: int, kv_heads: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """`rope_cache` and `decode_attention` of ONE new token per batch row in one launch: qkv
    [B, 1, q_heads + 2 kv_heads, hd] un-rotated (and left so); the rotated key and the value are written
    into the caches at pos [1]; returns [B, q_heads * hd].  Bit-identical to the two separate calls."""
    B, T, H, hd = qkv.shape
    assert T == 1 and H == q_heads + 2 * kv_heads and qkv.is_contiguous() and qkv.dtype == torch.float16
    assert pos.dtype == torch.int64 and pos.numel() == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape == v_cache.shape == (B, kv_heads, k_cache.shape[2], hd)
    assert cos.dtype == sin.dtype == torch.float16 and cos.is_contiguous() and sin.is_contiguous()
    if out is None:
        out = torch.empty(B, q_heads * hd, dtype=torch.float16, device=qkv.device)
    _native.check(_native.lib().qfb_decode_attention_rope(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(),
                                                          k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), B, q_heads,
                                                          kv_heads, hd, k_cache.shape[2], _stream(qkv)),
                  "qfb_decode_attention_rope")
    return out
