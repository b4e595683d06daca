"""The quantized decoder against the same network evaluated with dequantised fp32 weights: the
weights the kernels' own decode path yields, and the weights the CPU oracle dequantises from the
codes, scales and zeros the layers were built from."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import qf_oracle as O
from qfactory.decoder import DecoderConfig, QuantDecoder, run_decode

pytestmark = pytest.mark.gpu


def _oracle_weight(t):
    """fp32 [K, N] on the GPU from (codes, scales, GPTQ zeros), dequantised by the CPU oracle."""
    q, s, z = (a.cpu() for a in t)
    return O.dequant_effective(q, s, O.effective_zero(z.numpy(), 4)).float().cuda()


def _reference_logits(model, tokens, weights=None):
    """`weights`: None = each layer's dequantize(); else a function (block index, name) -> fp32 [K, N]."""
    cfg = model.cfg
    B, T = tokens.shape
    pos = torch.arange(T, device=tokens.device)
    x = model.embed[tokens].float()
    rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    for bi, blk in enumerate(model.blocks):
        if weights is None:
            W = lambda l: l.dequantize().float()       # [K, N] through the kernels' own decode path
        else:
            W = lambda l, bi=bi, blk=blk: weights(bi, {id(blk.qkv): "qkv", id(blk.o): "o", id(blk.gate_up): "gate_up",
                                                        id(blk.down): "down"}[id(l)])
        h = rms(x, blk.norm1)
        qkv = (h.view(B * T, -1) @ W(blk.qkv)).view(B, T, blk.hq + 2 * blk.hkv, blk.hd)
        q, k, v = qkv[:, :, : blk.hq], qkv[:, :, blk.hq : blk.hq + blk.hkv], qkv[:, :, blk.hq + blk.hkv :]
        rope = lambda t: model._rope(t.half(), pos).float()
        q, k = rope(q), rope(k)
        att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                             enable_gqa=True)
        x = x + (att.transpose(1, 2).reshape(B * T, -1) @ W(blk.o)).view(B, T, -1)
        h = rms(x, blk.norm2)
        gu = h.view(B * T, -1) @ W(blk.gate_up)
        half = gu.shape[-1] // 2
        x = x + ((F.silu(gu[:, :half]) * gu[:, half:]) @ W(blk.down)).view(B, T, -1)
    head = model.lm_head.dequantize().float() if weights is None else weights(-1, "lm_head")
    return rms(x[:, -1], model.final_norm) @ head


def test_small_decoder_matches_dequantised_reference():
    cfg = DecoderConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64)
    model = QuantDecoder(cfg, world=1, rank=0, device="cuda", seed=1, batch=2)
    # scales large enough for the linears to matter
    for blk in model.blocks:
        for l in (blk.qkv, blk.o, blk.gate_up, blk.down):
            l.s.mul_(40.0)
    tokens = torch.randint(0, cfg.vocab, (2, 9), device="cuda")
    with torch.no_grad():
        got = model(tokens, torch.arange(9, device="cuda")).float()
        want = _reference_logits(model, tokens)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()


def test_graph_decode_equals_eager_decode():
    cfg = DecoderConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64)
    a = QuantDecoder(cfg, device="cuda", seed=2, batch=1)
    b = QuantDecoder(cfg, device="cuda", seed=2, batch=1)
    _, ta = run_decode(a, prompt_len=8, steps=6, use_graph=True, seed=3)
    _, tb = run_decode(b, prompt_len=8, steps=6, use_graph=False, seed=3)
    assert torch.equal(ta, tb)


def test_seeded_decoder_matches_the_oracle_dequantised_network():
    """Weights drawn as codes / scales / zeros (the form the tensor-parallel ranks shard): the
    reference network is built from the ORACLE's dequantisation of those tensors."""
    cfg = DecoderConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64)
    model = QuantDecoder(cfg, world=1, rank=0, device="cuda", seed=4, batch=2, weights="seeded_keep")
    boost = lambda t: (t[0], (t[1].float() * 40.0).half(), t[2])     # scales large enough for the linears to matter
    for blk in model.blocks:
        blk.full = {k: boost(v) for k, v in blk.full.items()}
        for l in (blk.qkv, blk.o, blk.gate_up, blk.down):
            l.s.mul_(40.0)

    def weights(bi, name):
        if name == "lm_head":
            return _oracle_weight(model.lm_head_full)
        f = model.blocks[bi].full
        if name == "qkv":
            return torch.cat([_oracle_weight(f[n]) for n in ("q", "k", "v")], dim=1)
        if name == "gate_up":
            return torch.cat([_oracle_weight(f[n]) for n in ("gate", "up")], dim=1)
        return _oracle_weight(f[name])

    tokens = torch.randint(0, cfg.vocab, (2, 9), device="cuda")
    with torch.no_grad():
        got = model(tokens, torch.arange(9, device="cuda")).float()
        want = _reference_logits(model, tokens, weights)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()


def test_fused_and_unfused_activation_give_the_same_tokens_and_logits():
    cfg = DecoderConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64, scale_boost=40.0)
    a = QuantDecoder(cfg, device="cuda", seed=5, batch=2, weights="seeded")
    b = QuantDecoder(cfg, device="cuda", seed=5, batch=2, weights="seeded")
    b.fuse_silu = False
    tok = torch.randint(0, cfg.vocab, (2, 1), device="cuda")
    pos = torch.zeros(1, dtype=torch.long, device="cuda")
    with torch.no_grad():
        assert torch.equal(a(tok, pos), b(tok, pos))   # the fused staging computes the same bits


def test_fused_and_unfused_norm_give_close_logits():
    """The add + norm folded into the QKV / gate+up / output projections (one fp16 rounding of the
    activations instead of two, 1 / rms applied to the result): logits within 3e-3 of the largest one over
    a prefill and several single-token steps."""
    cfg = DecoderConfig(layers=3, d_model=512, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64, scale_boost=40.0)
    a = QuantDecoder(cfg, device="cuda", seed=7, batch=2, weights="seeded")
    b = QuantDecoder(cfg, device="cuda", seed=7, batch=2, weights="seeded")
    a.fuse_norm, b.fuse_norm = True, False
    tokens = torch.randint(0, cfg.vocab, (2, 12), device="cuda")
    from qfactory.decoder import teacher_forced_logits

    la = teacher_forced_logits(a, tokens, 6).float()
    lb = teacher_forced_logits(b, tokens, 6).float()
    assert torch.isfinite(la).all()
    assert (la - lb).abs().max() <= 3e-3 * lb.abs().max()
