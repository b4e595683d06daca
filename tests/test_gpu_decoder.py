"""The quantized decoder against the same network evaluated with dequantised fp32 weights."""
import pytest
import torch
import torch.nn.functional as F

from qfactory.decoder import DecoderConfig, QuantDecoder, run_decode

pytestmark = pytest.mark.gpu


def _reference_logits(model, tokens):
    cfg = model.cfg
    B, T = tokens.shape
    pos = torch.arange(T, device=tokens.device)
    x = model.embed[tokens].float()
    rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    for blk in model.blocks:
        W = lambda l: l.dequantize().float()       # [K, N] through the kernels' own decode path
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
    return rms(x[:, -1], model.final_norm) @ model.lm_head.float()


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
