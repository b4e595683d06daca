"""A small tensor-parallel Llama-architecture decoder whose linears are all quantized.

This is the end-to-end workload of the decode benchmark: random-init weights of the
Llama-2-70B architecture (80 layers, d = 8192, 64 query heads / 8 KV heads, FFN 28672,
vocab 32000), every linear W4A16 g128.  The sharding follows the reference's serve path
(reference: third_party/vllm-bitblas/vllm/model_executor/models/llama.py:60-285 with
layers/linear.py:382-394, 1100-1124): fused QKV and gate+up are column-parallel (no
collective), O and down are row-parallel followed by ONE all-reduce each.  RMSNorm, SiLU * up and
RoPE with the cache write are one native launch each (ops.py; `native_ops=False` keeps the plain
torch expressions, which the tests compare against); attention is torch's SDPA.

Weights are random packed bytes generated on the device (the reference's own end-to-end
runs also used uninitialised weights, third_party/vllm-qfactory.patch:223-228).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _native, ops
from .parallel import all_reduce_sum
from .qlinear import QLinear


@dataclass
class DecoderConfig:
    layers: int = 80
    d_model: int = 8192
    n_heads: int = 64
    n_kv_heads: int = 8
    d_ff: int = 28672
    vocab: int = 32000
    bits: int = 4
    group_size: int = 128
    max_len: int = 512
    rope_theta: float = 10000.0

    @property
    def head_dim(self):
        return self.d_model // self.n_heads


def _random_layer(K, N, bits, gs, device, gen, batch=1):
    # the batch the decoder is built for picks the packed layout (fragment up to 16 rows)
    L = QLinear.empty(batch, K, N, bits, gs, sym=False, device=device)
    L.w.copy_(torch.randint(-128, 128, L.w.shape, generator=gen, dtype=torch.int8, device=device))
    # small scales keep the residual stream of a random-weight network finite
    L.s.copy_((torch.rand(L.s.shape, generator=gen, device=device) * 2e-4 + 1e-4).half())
    L.z.copy_(torch.randint(7, 10, L.z.shape, generator=gen, dtype=torch.int8, device=device))
    # programmatic dependent launch: the layer's weight prefetch overlaps the tail of whatever ran before
    L.flags = _native.FLAG_PDL
    return L


class DecoderLayer(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, world: int, device, gen, batch: int = 1):
        super().__init__()
        d, hd = cfg.d_model, cfg.head_dim
        self.hq, self.hkv, self.hd = cfg.n_heads // world, cfg.n_kv_heads // world, hd
        self.qkv = _random_layer(d, (self.hq + 2 * self.hkv) * hd, cfg.bits, cfg.group_size, device, gen, batch)   # column parallel
        self.o = _random_layer(self.hq * hd, d, cfg.bits, cfg.group_size, device, gen, batch)                       # row parallel
        self.gate_up = _random_layer(d, 2 * cfg.d_ff // world, cfg.bits, cfg.group_size, device, gen, batch)        # column parallel
        self.down = _random_layer(cfg.d_ff // world, d, cfg.bits, cfg.group_size, device, gen, batch)               # row parallel
        self.norm1 = torch.nn.Parameter(torch.ones(d, dtype=torch.float16, device=device), requires_grad=False)
        self.norm2 = torch.nn.Parameter(torch.ones(d, dtype=torch.float16, device=device), requires_grad=False)


class QuantDecoder(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, world: int = 1, rank: int = 0, device="cuda", seed: int = 0, batch: int = 1,
                 native_ops: bool = True):
        super().__init__()
        self.native_ops = native_ops
        assert cfg.n_kv_heads % world == 0 and cfg.d_ff % (world * cfg.group_size) == 0
        self.cfg, self.world, self.rank, self.batch = cfg, world, rank, batch
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
        self.blocks = torch.nn.ModuleList([DecoderLayer(cfg, world, device, gen, batch) for _ in range(cfg.layers)])
        g0 = torch.Generator(device=device).manual_seed(seed)  # replicated tensors: same on every rank
        self.embed = (torch.randn(cfg.vocab, cfg.d_model, generator=g0, device=device) * 0.02).half()
        self.lm_head = (torch.randn(cfg.d_model, cfg.vocab, generator=g0, device=device) * 0.02).half()
        self.final_norm = torch.ones(cfg.d_model, dtype=torch.float16, device=device)
        hd = cfg.head_dim
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=device).float() / hd))
        ang = torch.arange(cfg.max_len, device=device).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().half(), ang.sin().half()
        hkv = cfg.n_kv_heads // world
        self.k_cache = torch.zeros(cfg.layers, batch, hkv, cfg.max_len, hd, dtype=torch.float16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)

    def _rms(self, x, w):
        if self.native_ops:
            return ops.rmsnorm(x.contiguous(), w, 1e-5)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w

    def _add_rms(self, x, r, w):
        """x += r in place, then the norm of the sum (one launch with the native ops)."""
        if self.native_ops:
            return ops.add_rmsnorm(x, r.contiguous(), w, 1e-5)
        x += r
        return self._rms(x, w)

    def _rope(self, t, pos):
        # t [B, T, H, hd]; pos [T] long
        c, s = self.cos[pos][None, :, None, :], self.sin[pos][None, :, None, :]
        t1, t2 = t[..., 0::2], t[..., 1::2]
        return torch.stack((t1 * c - t2 * s, t1 * s + t2 * c), dim=-1).flatten(-2)

    def forward(self, tokens: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] long, pos [T] long positions (device tensor, so that a captured graph can
        be replayed with new positions).  Returns logits of the last position [B, vocab]."""
        cfg = self.cfg
        B, T = tokens.shape
        x = self.embed[tokens]                                   # [B, T, d]
        mask = None   # built on first use: the single-token step with the native attention needs none
        pending = None   # output of the previous down projection, not yet added to the residual stream
        for li, blk in enumerate(self.blocks):
            h = self._add_rms(x, pending, blk.norm1) if pending is not None else self._rms(x, blk.norm1)
            qkv = blk.qkv(h.view(B * T, -1)).view(B, T, blk.hq + 2 * blk.hkv, blk.hd)
            q, k, v = qkv[:, :, : blk.hq], qkv[:, :, blk.hq : blk.hq + blk.hkv], qkv[:, :, blk.hq + blk.hkv :]
            if self.native_ops:
                ops.rope_cache(qkv, self.cos, self.sin, pos, self.k_cache[li], self.v_cache[li], blk.hq, blk.hkv)
            else:
                q, k = self._rope(q, pos), self._rope(k, pos)
                self.k_cache[li].index_copy_(2, pos, k.transpose(1, 2))
                self.v_cache[li].index_copy_(2, pos, v.transpose(1, 2))
            if self.native_ops and T == 1 and ops.decode_attention_supported(blk.hq, blk.hkv, blk.hd, cfg.max_len):
                att2d = ops.decode_attention(qkv, pos, self.k_cache[li], self.v_cache[li], blk.hq, blk.hkv)   # [B, hq * hd]
            else:
                if mask is None:
                    # causal mask over the whole static cache: key j visible to query i iff j <= pos[i]
                    mask = torch.arange(cfg.max_len, device=x.device)[None, :] <= pos[:, None]   # [T, max_len]
                att = F.scaled_dot_product_attention(q.transpose(1, 2), self.k_cache[li], self.v_cache[li],
                                                     attn_mask=mask[None, None], enable_gqa=True)   # [B, hq, T, hd]
                att2d = att.transpose(1, 2).reshape(B * T, -1)
            o = blk.o(att2d)
            all_reduce_sum(o)                                     # row parallel
            h = self._add_rms(x, o.view(B, T, -1), blk.norm2)     # x += o, then the norm
            gu = blk.gate_up(h.view(B * T, -1))
            half = gu.shape[-1] // 2
            act = ops.silu_mul(gu) if self.native_ops else F.silu(gu[:, :half]) * gu[:, half:]
            dn = blk.down(act)
            all_reduce_sum(dn)                                    # row parallel
            pending = dn.view(B, T, -1)                           # added by the next layer's (or the final) norm
        x = x + pending
        last = self._rms(x[:, -1], self.final_norm)
        return last @ self.lm_head


def quantized_bytes_per_token(cfg: DecoderConfig, world: int = 1) -> int:
    """Packed weight + scale + zero bytes one rank streams per decoded token."""
    d, hd = cfg.d_model, cfg.head_dim
    shapes = [((cfg.n_heads + 2 * cfg.n_kv_heads) * hd // world, d), (d, cfg.n_heads * hd // world),
              (2 * cfg.d_ff // world, d), (d, cfg.d_ff // world)]
    per = sum(n * k * cfg.bits // 8 + (k // cfg.group_size) * n * 3 for n, k in shapes)
    return per * cfg.layers


def run_decode(model: QuantDecoder, prompt_len: int = 128, steps: int = 256, use_graph: bool = True, seed: int = 0):
    """Prefill `prompt_len` uniform-random token ids, then greedy-decode `steps` tokens.
    Returns (decode seconds on the device, last tokens [B]).  The decode step is captured in a
    CUDA graph (static cache, position passed as a device tensor); collectives are NCCL."""
    cfg, B = model.cfg, model.batch
    dev = model.embed.device
    assert prompt_len + steps <= cfg.max_len
    g = torch.Generator(device=dev).manual_seed(seed)
    prompt = torch.randint(0, cfg.vocab, (B, prompt_len), generator=g, device=dev)
    with torch.no_grad():
        logits = model(prompt, torch.arange(prompt_len, device=dev))
        tok = logits.argmax(-1, keepdim=True)                   # [B, 1]
        pos = torch.full((1,), prompt_len, dtype=torch.long, device=dev)
        graph = None
        if use_graph:
            s = torch.cuda.Stream(device=dev)
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):
                for _ in range(2):                              # warm up outside capture
                    model(tok, pos)
            torch.cuda.current_stream(dev).wait_stream(s)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out_logits = model(tok, pos)
                next_tok = out_logits.argmax(-1, keepdim=True)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            if graph is not None:
                graph.replay()
                tok.copy_(next_tok)
            else:
                tok = model(tok, pos).argmax(-1, keepdim=True)
            pos += 1
        e1.record()
        torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) * 1e-3, tok.flatten()
