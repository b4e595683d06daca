"""A small tensor-parallel Llama-architecture decoder whose linears are all quantized.

This is the end-to-end workload of the decode benchmark: random-init weights of the
Llama-2-70B architecture (80 layers, d = 8192, 64 query heads / 8 KV heads, FFN 28672,
vocab 32000), every linear W4A16 g128.  The sharding follows the reference's serve path
(reference: third_party/vllm-bitblas/vllm/model_executor/models/llama.py:60-285 with
layers/linear.py:382-394, 1100-1124): fused QKV and gate+up are column-parallel (no
collective), O and down are row-parallel followed by ONE all-reduce each.  RMSNorm, SiLU * up,
RoPE with the cache write and the single-token attention are one native launch each (ops.py;
`native_ops=False` keeps the plain torch expressions, which the tests compare against); the
prefill's attention is torch's SDPA.

The all-reduce of a decode step (at most 64 rows) is the library's one-shot peer-memory kernel,
fused with the residual add and the RMS norm that follow it (comm.py): the row-parallel linear
writes its partial into the communicator's slot, one launch does the rest.  Larger row counts (a
prefill) use the process group's all-reduce (NCCL), as does everything when `collective='nccl'`.

Weights: `weights='packed'` draws random packed bytes on the device (the reference's own
end-to-end runs also used uninitialised weights, third_party/vllm-qfactory.patch:223-228);
`weights='seeded'` draws ONE set of codes / scales / zeros from the seed, the same on every rank,
and each rank packs its column or row shard of it (parallel.py), so that a tensor-parallel model
is the same network as the single-GPU one and their outputs can be compared.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _native, ops
from .parallel import all_reduce_sum, shard_columns, shard_rows
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
    scale_boost: float = 1.0   # multiplies the (small) random scales: >1 makes the linears matter in numeric checks

    @property
    def head_dim(self):
        return self.d_model // self.n_heads


def _random_layer(K, N, bits, gs, device, gen, batch=1, boost=1.0):
    # the batch the decoder is built for picks the packed layout (fragment up to 16 rows)
    L = QLinear.empty(batch, K, N, bits, gs, sym=False, device=device)
    L.w.copy_(torch.randint(-128, 128, L.w.shape, generator=gen, dtype=torch.int8, device=device))
    # small scales keep the residual stream of a random-weight network finite
    L.s.copy_(((torch.rand(L.s.shape, generator=gen, device=device) * 2e-4 + 1e-4) * boost).half())
    L.z.copy_(torch.randint(7, 10, L.z.shape, generator=gen, dtype=torch.int8, device=device))
    # programmatic dependent launch: the layer's weight prefetch overlaps the tail of whatever ran before
    L.flags = _native.FLAG_PDL
    return L


def seeded_tensors(K, N, bits, gs, gen, device, boost=1.0):
    """Codes [K,N], scales [K/gs,N], GPTQ-convention zeros [K/gs,N] of one full (unsharded) linear,
    drawn on `device` from `gen`; the distributions keep the residual stream of a random network finite."""
    q = torch.randint(0, 1 << bits, (K, N), generator=gen, dtype=torch.int32, device=device)
    s = ((torch.rand(K // gs, N, generator=gen, device=device) * 2e-4 + 1e-4) * boost).half()
    z = torch.randint((1 << bits) // 2 - 2, (1 << bits) // 2 + 1, (K // gs, N), generator=gen, dtype=torch.int32, device=device)
    return q, s, z


def _packed(K, N, cfg, parts, batch):
    """QLinear of the column-wise concatenation of (codes, scales, zeros) parts."""
    q = torch.cat([p[0] for p in parts], dim=1)
    s = torch.cat([p[1] for p in parts], dim=1)
    z = torch.cat([p[2] for p in parts], dim=1)
    L = QLinear.init(batch, K, N, cfg.bits, q, cfg.group_size, s, z)
    L.flags = _native.FLAG_PDL
    return L


class DecoderLayer(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, world: int, device, gen, batch: int = 1, weights: str = "packed", rank: int = 0):
        super().__init__()
        d, hd = cfg.d_model, cfg.head_dim
        self.hq, self.hkv, self.hd = cfg.n_heads // world, cfg.n_kv_heads // world, hd
        nq, nkv, ff = cfg.n_heads * hd, cfg.n_kv_heads * hd, cfg.d_ff
        if weights == "packed":
            self.qkv = _random_layer(d, (self.hq + 2 * self.hkv) * hd, cfg.bits, cfg.group_size, device, gen, batch, cfg.scale_boost)   # column parallel
            self.o = _random_layer(self.hq * hd, d, cfg.bits, cfg.group_size, device, gen, batch, cfg.scale_boost)                       # row parallel
            self.gate_up = _random_layer(d, 2 * cfg.d_ff // world, cfg.bits, cfg.group_size, device, gen, batch, cfg.scale_boost)        # column parallel
            self.down = _random_layer(cfg.d_ff // world, d, cfg.bits, cfg.group_size, device, gen, batch, cfg.scale_boost)               # row parallel
        else:
            # the full tensors of the layer, identical on every rank; this rank keeps its shards:
            # the query / key / value (gate / up) column shards are fused, O and down are split along K
            T = lambda K, N: seeded_tensors(K, N, cfg.bits, cfg.group_size, gen, device, cfg.scale_boost)
            col = lambda t: shard_columns(*t, rank, world)
            row = lambda t: shard_rows(*t, rank, world, cfg.group_size)
            full = {}
            for name, (K_, N_) in (("q", (d, nq)), ("k", (d, nkv)), ("v", (d, nkv)), ("o", (nq, d)), ("gate", (d, ff)),
                                   ("up", (d, ff)), ("down", (ff, d))):
                full[name] = T(K_, N_)     # drawn in this fixed order on every rank
            tq, tk, tv, to, tg, tu, td = (full[n] for n in ("q", "k", "v", "o", "gate", "up", "down"))
            self.full = full if weights == "seeded_keep" else None
            self.qkv = _packed(d, (self.hq + 2 * self.hkv) * hd, cfg, [col(tq), col(tk), col(tv)], batch)
            self.o = _packed(nq // world, d, cfg, [row(to)], batch)
            self.gate_up = _packed(d, 2 * ff // world, cfg, [col(tg), col(tu)], batch)
            self.down = _packed(ff // world, d, cfg, [row(td)], batch)
        self.norm1 = torch.nn.Parameter(torch.ones(d, dtype=torch.float16, device=device), requires_grad=False)
        self.norm2 = torch.nn.Parameter(torch.ones(d, dtype=torch.float16, device=device), requires_grad=False)


class QuantDecoder(torch.nn.Module):
    """`collective`: 'auto' (the peer-memory kernel for decode steps when a process group with more
    than one rank exists, NCCL otherwise), 'nccl' (the process group's all-reduce everywhere) or
    'none' (no reduction at all: an ablation for timing, the outputs are then wrong for world > 1).
    `weights`: 'packed' | 'seeded' | 'seeded_keep' (as 'seeded', and the layers keep the full tensors
    in `.full` for reference computations)."""

    def __init__(self, cfg: DecoderConfig, world: int = 1, rank: int = 0, device="cuda", seed: int = 0, batch: int = 1,
                 native_ops: bool = True, weights: str = "packed", collective: str = "auto"):
        super().__init__()
        self.native_ops = native_ops
        self.fuse_silu = True   # False: SiLU * up as a launch of its own (tests compare the two)
        self.fuse_rope = True   # False: rotary embedding + cache write as a launch of its own before the attention
        self.fuse_push = True   # False: the row-parallel linears only store their partial; the reduction kernel sends it
        # True: residual add + RMS norm folded into QKV / gate+up / the head (QLinear.forward_addnorm) instead of a
        # launch of their own.  Off: inside a CUDA graph the small norm launch already hides behind the next
        # linear's weight prefetch (programmatic dependent launch), and the fused staging was measured 2 % slower
        # per token (9.23 against 9.05 ms); it pays where launches are issued one by one.
        self.fuse_norm = False
        # True (tensor-parallel decode steps): no reduction kernel between a row-parallel linear and the linear that
        # consumes its sum: O / down send their partials themselves, and gate+up / the next QKV collect them, add
        # them to the residual stream and apply the norm while they stage their activations (step-numbered
        # epochs, PeerComm.step_begin).  Only the last reduction of a step (final norm) is a launch of its own.
        # Off: measured 10 % slower per token at two ranks (6.49 against 5.84-5.90 ms): every CTA of the consuming
        # GEMV polls and sums its slice (the work of one small kernel repeated per row tile, on the GEMV's own
        # latency chain), which costs more than the launch it saves.
        self.fuse_collect = False
        assert cfg.n_kv_heads % world == 0 and cfg.d_ff % (world * cfg.group_size) == 0
        assert weights in ("packed", "seeded", "seeded_keep") and collective in ("auto", "nccl", "none")
        self.cfg, self.world, self.rank, self.batch = cfg, world, rank, batch
        self.collective = collective
        # packed bytes differ per rank (they are that rank's shard of some network); seeded tensors
        # are the whole network, drawn identically everywhere
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + (rank if weights == "packed" else 0))
        self.blocks = torch.nn.ModuleList([DecoderLayer(cfg, world, device, gen, batch, weights, rank) for _ in range(cfg.layers)])
        g0 = torch.Generator(device=device).manual_seed(seed)  # replicated tensors: same on every rank
        self.embed = (torch.randn(cfg.vocab, cfg.d_model, generator=g0, device=device) * 0.02).half()
        # the output projection is a quantized linear like the others (replicated: 0.13 GB at 4 bits)
        if weights == "packed":
            self.lm_head = _random_layer(cfg.d_model, cfg.vocab, cfg.bits, cfg.group_size, device, g0, batch)
            self.lm_head.s.mul_(100.0)
            self.lm_head_full = None
        else:
            t = seeded_tensors(cfg.d_model, cfg.vocab, cfg.bits, cfg.group_size, g0, device)
            t = (t[0], (t[1].float() * 100.0).half(), t[2])
            self.lm_head = _packed(cfg.d_model, cfg.vocab, cfg, [t], batch)
            self.lm_head_full = t if weights == "seeded_keep" else None
        self.final_norm = torch.ones(cfg.d_model, dtype=torch.float16, device=device)
        hd = cfg.head_dim
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=device).float() / hd))
        ang = torch.arange(cfg.max_len, device=device).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().half(), ang.sin().half()
        hkv = cfg.n_kv_heads // world
        self.k_cache = torch.zeros(cfg.layers, batch, hkv, cfg.max_len, hd, dtype=torch.float16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        # peer-memory communicator for the reductions of a decode step
        self.comm, self.comm_error = None, None
        if world > 1 and collective == "auto":
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                try:
                    from .comm import PeerComm

                    self.comm = PeerComm.from_process_group(cfg.d_model, 64, torch.device(device))
                    self.comm.set_timeout_us(500_000)   # ranks of one node are never this far apart inside a step
                except Exception as e:  # peers not mappable (no peer access, IPC closed): NCCL serves every reduction
                    self.comm_error = str(e)[:160]
                # all ranks must agree, or their call sequences diverge
                ok = torch.tensor([1 if self.comm is not None else 0], device=device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if int(ok[0]) == 0 and self.comm is not None:
                    self.comm.close()
                    self.comm, self.comm_error = None, "a peer could not map the buffers"

    def collective_name(self):
        if self.world == 1:
            return "none"
        if self.collective == "none":
            return "none (ablation)"
        if self.comm is not None:
            return "one-shot peer-memory all-reduce fused with add + rmsnorm (decode), nccl (prefill)"
        return "nccl all_reduce after O and down" + (f" (peer setup failed: {self.comm_error})" if self.comm_error else "")

    def _reduce(self, t):
        if self.collective != "none":
            all_reduce_sum(t)

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

    def _norm_linear(self, lin, cur, r, w, spare):
        """y = lin(rmsnorm(cur + r) * w) for the residual stream `cur` [rows, d] (`r` may be None).  Returns
        (y, the tensor that now holds cur + r, the other of the two buffers).  One kernel where the fused
        form serves the layer and the batch (`QLinear.forward_addnorm`: it writes the sum into `spare`,
        because other blocks of the launch still read `cur`); otherwise the add + norm launch, in place
        on `cur`, then the linear."""
        if self.fuse_norm and self.native_ops:
            y = lin.forward_addnorm(cur, r, w, 1e-5, x_out=spare if r is not None else None)
            if y is not None:
                return (y, spare, cur) if r is not None else (y, cur, spare)
        h = self._add_rms(cur, r, w) if r is not None else self._rms(cur, w)
        return lin(h), cur, spare

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
        R = B * T
        x = self.embed[tokens]                                   # [B, T, d], contiguous
        x2 = x.view(R, -1)
        fused = self.comm is not None and self.collective == "auto" and self.native_ops and self.comm.fits(R, cfg.d_model)
        mask = None   # built on first use: the single-token step with the native attention needs none
        pending = None   # output of the previous down projection, not yet added to the residual stream
        h = None         # fused path: the normed input of the next layer, made by the reduction kernel
        nblk = len(self.blocks)
        # the collecting form of the communicator path: every reduction of the step but the last is received by the
        # GEMV that consumes it
        blk0 = self.blocks[0]
        collect = (fused and self.fuse_collect and self.fuse_push and T == 1 and 2 * nblk <= 256
                   and self.comm.collect_supported(blk0.o, blk0.gate_up, R) and self.comm.collect_supported(blk0.down, blk0.qkv, R)
                   and (not self.fuse_silu or blk0.down.silu_mul_supported(R)))
        if collect:
            self.comm.step_begin()
        # without the reduction kernel the residual stream lives in two buffers used in turn (see _norm_linear)
        cur, spare = x2, (torch.empty_like(x2) if (collect or not fused) else None)
        for li, blk in enumerate(self.blocks):
            if collect:
                if li == 0:
                    qkv2d = blk.qkv(self._rms(x2, blk.norm1))
                else:   # residual += sum of the previous down projection's partials (slot 1), norm 1, QKV: one launch
                    qkv2d = self.comm.collect_norm_linear(blk.qkv, 1, 2 * li - 1, cur, spare, blk.norm1, R)
                    cur, spare = spare, cur
            elif fused:
                if h is None:
                    h = self._rms(x2, blk.norm1)          # first layer; afterwards the reduction kernel makes it
                qkv2d = blk.qkv(h.view(R, -1))
            else:
                qkv2d, cur, spare = self._norm_linear(blk.qkv, cur, pending, blk.norm1, spare)
            qkv = qkv2d.view(B, T, blk.hq + 2 * blk.hkv, blk.hd)
            q, k, v = qkv[:, :, : blk.hq], qkv[:, :, blk.hq : blk.hq + blk.hkv], qkv[:, :, blk.hq + blk.hkv :]
            native_attn = self.native_ops and T == 1 and ops.decode_attention_supported(blk.hq, blk.hkv, blk.hd, cfg.max_len)
            if native_attn and self.fuse_rope:
                # one launch: rotary embedding of the queries and the new key, cache write, attention
                att2d = ops.decode_attention_rope(qkv, self.cos, self.sin, pos, self.k_cache[li], self.v_cache[li],
                                                  blk.hq, blk.hkv)                                            # [B, hq * hd]
            else:
                if self.native_ops:
                    ops.rope_cache(qkv, self.cos, self.sin, pos, self.k_cache[li], self.v_cache[li], blk.hq, blk.hkv)
                else:
                    q, k = self._rope(q, pos), self._rope(k, pos)
                    self.k_cache[li].index_copy_(2, pos, k.transpose(1, 2))
                    self.v_cache[li].index_copy_(2, pos, v.transpose(1, 2))
                if native_attn:
                    att2d = ops.decode_attention(qkv, pos, self.k_cache[li], self.v_cache[li], blk.hq, blk.hkv)   # [B, hq * hd]
                else:
                    if mask is None:
                        # causal mask over the whole static cache: key j visible to query i iff j <= pos[i]
                        mask = torch.arange(cfg.max_len, device=x.device)[None, :] <= pos[:, None]   # [T, max_len]
                    att = F.scaled_dot_product_attention(q.transpose(1, 2), self.k_cache[li], self.v_cache[li],
                                                         attn_mask=mask[None, None], enable_gqa=True)   # [B, hq, T, hd]
                    att2d = att.transpose(1, 2).reshape(R, -1)
            if collect:
                # O sends its partial (reduction 2 li, slot 0); gate+up collects it: residual += sum, norm 2, gate/up
                self.comm.linear_into_slot(blk.o, att2d, 0, R, idx=2 * li)
                gu = self.comm.collect_norm_linear(blk.gate_up, 0, 2 * li, cur, spare, blk.norm2, R)
                cur, spare = spare, cur
            elif fused:
                # row parallel: the partial goes straight into the communicator's slot; ONE launch then
                # sums it over the ranks, adds it to the residual stream and applies the next norm
                pushed = self.comm.linear_into_slot(blk.o, att2d, 0, R, push=self.fuse_push)
                h = self.comm.allreduce_add_rmsnorm(0, x2, blk.norm2, R, pushed=pushed)
                gu = blk.gate_up(h.view(R, -1))
            else:
                o = blk.o(att2d)
                self._reduce(o)                                       # row parallel
                gu, cur, spare = self._norm_linear(blk.gate_up, cur, o, blk.norm2, spare)   # residual += o, norm, gate/up
            half = gu.shape[-1] // 2
            # SiLU(gate) * up is combined inside the down projection's activation staging where that
            # kernel serves the batch (`down` below); otherwise as a launch of its own
            fuse_act = self.native_ops and self.fuse_silu and blk.down.silu_mul_supported(R)
            if fuse_act:
                down = lambda out=None: blk.down.forward_silu_mul(gu, out=out)
            else:
                act = ops.silu_mul(gu) if self.native_ops else F.silu(gu[:, :half]) * gu[:, half:]
                down = lambda out=None: blk.down(act, out=out)
            if collect:
                # down sends its partial (reduction 2 li + 1, slot 1); the next layer's QKV collects it, or, after
                # the last layer, the reduction kernel with the final norm
                self.comm.linear_into_slot(blk.down, gu if fuse_act else act, 1, R, silu_mul=fuse_act, idx=2 * li + 1)
                if li + 1 == nblk:
                    h = self.comm.allreduce_add_rmsnorm(1, cur, self.final_norm, R, idx=2 * li + 1)
            elif fused:
                pushed = self.comm.linear_into_slot(blk.down, gu if fuse_act else act, 1, R, silu_mul=fuse_act,
                                                    push=self.fuse_push)
                last = li + 1 == nblk
                if not last:
                    h = self.comm.allreduce_add_rmsnorm(1, x2, self.blocks[li + 1].norm1, R, pushed=pushed)
                elif T == 1:
                    h = self.comm.allreduce_add_rmsnorm(1, x2, self.final_norm, R, pushed=pushed)   # the final norm of every row
                else:
                    self.comm.allreduce_add_rmsnorm(1, x2, None, R, out=x2, pushed=pushed)          # x += sum; the final norm follows
                    h = None
                pending = None
            else:
                dn = down()
                self._reduce(dn)                                      # row parallel
                pending = dn                                          # added by the next layer's (or the final) norm
        if fused:
            last = h.view(B, -1) if T == 1 else self._rms(x[:, -1], self.final_norm)
            return self.lm_head(last)
        if T == 1:
            return self._norm_linear(self.lm_head, cur, pending, self.final_norm, spare)[0]
        if pending is not None:
            cur = cur + pending
        return self.lm_head(self._rms(cur.view(B, T, -1)[:, -1].contiguous(), self.final_norm))

    def close(self):
        if self.comm is not None:
            self.comm.close()
            self.comm = None


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
                for i in range(2):                              # warm up outside capture
                    model(tok, pos)
                    if i == 0 and model.comm is not None:
                        # a wait that ran out in the first step: every rank drops to the process group's
                        # all-reduce before anything is captured
                        import torch.distributed as dist

                        torch.cuda.synchronize(dev)
                        bad = torch.tensor([model.comm.read_status()], device=dev)
                        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                        if int(bad[0]) != 0:
                            model.close()
                            model.comm_error = "a bounded wait ran out in the warm-up step"
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


def teacher_forced_logits(model: QuantDecoder, tokens: torch.Tensor, prompt_len: int) -> torch.Tensor:
    """Logits after feeding `tokens` [B, L]: the first `prompt_len` as one prefill, the rest one at a
    time (eager launches, no graph).  Two models given the same tokens can be compared on the result
    without their greedy choices drifting apart."""
    dev = model.embed.device
    L = tokens.shape[1]
    assert L <= model.cfg.max_len and 0 < prompt_len <= L
    with torch.no_grad():
        logits = model(tokens[:, :prompt_len].contiguous(), torch.arange(prompt_len, device=dev))
        for t in range(prompt_len, L):
            logits = model(tokens[:, t : t + 1].contiguous(), torch.full((1,), t, dtype=torch.long, device=dev))
    torch.cuda.synchronize(dev)
    return logits


def time_linears(model: QuantDecoder, reps: int = 3) -> float:
    """Device seconds of the quantized linears of ONE decode step alone: every layer's four linears
    and the output projection, launched back to back from a CUDA graph on inputs of the decode
    step's shapes (each layer streams its own weights, as in the step)."""
    cfg, B, dev = model.cfg, model.batch, model.embed.device
    blk0 = model.blocks[0]
    with torch.no_grad():
        h = torch.randn(B, cfg.d_model, device=dev).half()
        att = torch.randn(B, blk0.hq * blk0.hd, device=dev).half()
        act = torch.randn(B, blk0.down.in_features, device=dev).half()
        outs = {id(l): torch.empty(B, l.out_features, dtype=torch.float16, device=dev)
                for l in (blk0.qkv, blk0.o, blk0.gate_up, blk0.down, model.lm_head)}

        def step():
            for blk in model.blocks:
                blk.qkv(h, out=outs[id(blk0.qkv)])
                blk.o(att, out=outs[id(blk0.o)])
                blk.gate_up(h, out=outs[id(blk0.gate_up)])
                blk.down(act, out=outs[id(blk0.down)])
            model.lm_head(h, out=outs[id(model.lm_head)])

        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            step()
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        g.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) * 1e-3 / reps
