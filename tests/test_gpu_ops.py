"""The element-wise neighbours of the linears (RMSNorm, SiLU * up, RoPE + cache write) against the
plain torch expressions they replace in the decoder."""
import pytest
import torch
import torch.nn.functional as F

from qfactory import ops
from qfactory.decoder import DecoderConfig, QuantDecoder

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,d", [(1, 8192), (3, 4096), (16, 512), (130, 1000)])
def test_rmsnorm_matches_the_torch_expression(rows, d):
    g = torch.Generator(device="cuda").manual_seed(rows + d)
    x = (torch.randn(rows, d, generator=g, device="cuda") * 3).half()
    w = (torch.rand(d, generator=g, device="cuda") + 0.5).half()
    xf = x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
    got = ops.rmsnorm(x, w, 1e-5)
    # the reduction order differs, so the fp32 reciprocal root may differ in its last bit: at most one
    # fp16 step on a few elements
    diff = (got.float() - want.float()).abs()
    assert (diff <= want.float().abs() * 2 ** -9 + 1e-6).all()
    assert (diff == 0).float().mean() > 0.98


@pytest.mark.parametrize("rows,half", [(1, 28672), (5, 11008), (16, 1024)])
def test_silu_mul_matches_the_torch_expression(rows, half):
    g = torch.Generator(device="cuda").manual_seed(half)
    gu = (torch.randn(rows, 2 * half, generator=g, device="cuda") * 2).half()
    want = F.silu(gu[:, :half]) * gu[:, half:]
    got = ops.silu_mul(gu)
    diff = (got.float() - want.float()).abs()
    assert (diff <= want.float().abs() * 2 ** -9 + 1e-6).all()   # the fast exponential: one fp16 step at most
    assert (diff == 0).float().mean() > 0.97


def test_rope_cache_is_bit_identical_to_the_torch_expression():
    B, T, hq, hkv, hd, L = 2, 5, 8, 2, 64, 32
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, T, hq + 2 * hkv, hd, generator=g, device="cuda").half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(L, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().half(), ang.sin().half()
    pos = torch.tensor([3, 4, 9, 10, 31], device="cuda")

    def rope(t):
        c, s = cos[pos][None, :, None, :], sin[pos][None, :, None, :]
        t1, t2 = t[..., 0::2], t[..., 1::2]
        return torch.stack((t1 * c - t2 * s, t1 * s + t2 * c), dim=-1).flatten(-2)

    q_want, k_want = rope(qkv[:, :, :hq]), rope(qkv[:, :, hq:hq + hkv])
    v_want = qkv[:, :, hq + hkv:].clone()
    kc = torch.zeros(B, hkv, L, hd, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    work = qkv.clone()
    ops.rope_cache(work, cos, sin, pos, kc, vc, hq, hkv)
    assert torch.equal(work[:, :, :hq], q_want) and torch.equal(work[:, :, hq:hq + hkv], k_want)
    assert torch.equal(work[:, :, hq + hkv:], v_want)
    assert torch.equal(kc[:, :, pos], k_want.transpose(1, 2)) and torch.equal(vc[:, :, pos], v_want.transpose(1, 2))
    untouched = torch.ones(L, dtype=torch.bool, device="cuda")
    untouched[pos] = False
    assert (kc[:, :, untouched] == 0).all() and (vc[:, :, untouched] == 0).all()


def test_decoder_with_native_ops_matches_decoder_with_torch_ops():
    cfg = DecoderConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64)
    a = QuantDecoder(cfg, device="cuda", seed=4, batch=2, native_ops=True)
    b = QuantDecoder(cfg, device="cuda", seed=4, batch=2, native_ops=False)
    for m in (a, b):
        for blk in m.blocks:
            for l in (blk.qkv, blk.o, blk.gate_up, blk.down):
                l.s.mul_(40.0)
    tokens = torch.randint(0, cfg.vocab, (2, 7), device="cuda")
    with torch.no_grad():
        ya = a(tokens, torch.arange(7, device="cuda")).float()
        yb = b(tokens, torch.arange(7, device="cuda")).float()
    assert torch.isfinite(ya).all()
    assert (ya - yb).abs().max() <= 5e-3 * yb.abs().max()
    assert (a.k_cache[:, :, :, :7].float() - b.k_cache[:, :, :, :7].float()).abs().max() <= 1e-2


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_native_quantizer_matches_the_reference_fixture(golden_dir, bits):
    import os

    import numpy as np

    from qfactory.quantize import asymmetric_quant

    f = np.load(os.path.join(golden_dir, f"quant_b{bits}.npz"))  # produced by the reference's own helper
    q, s, z = asymmetric_quant(torch.from_numpy(f["w"]).cuda(), int(f["GS"]), bits)
    assert np.array_equal(q.cpu().numpy(), f["q"])
    assert np.array_equal(s.cpu().numpy().view(np.uint16), f["s"].view(np.uint16))
    assert np.array_equal(z.cpu().numpy(), f["z"])


@pytest.mark.parametrize("bits,GS,K,N", [(4, 128, 1024, 300), (3, 128, 512, 64), (8, 64, 256, 1000), (2, 256, 512, 17)])
def test_native_quantizer_matches_the_torch_expression(bits, GS, K, N):
    from qfactory.quantize import asymmetric_quant

    g = torch.Generator().manual_seed(bits * 1000 + K)
    w = (torch.randn(K, N, generator=g) * 0.05).half()
    q0, s0, z0 = asymmetric_quant(w, GS, bits)            # CPU: the vectorised torch expression
    q1, s1, z1 = asymmetric_quant(w.cuda(), GS, bits)     # CUDA: the native kernel
    assert torch.equal(q1.cpu(), q0) and torch.equal(z1.cpu(), z0)
    assert torch.equal(s1.cpu().view(torch.int16), s0.view(torch.int16))


def test_add_rmsnorm_adds_in_place_and_norms_the_sum():
    g = torch.Generator(device="cuda").manual_seed(8)
    x = torch.randn(5, 4096, generator=g, device="cuda").half()
    r = torch.randn(5, 4096, generator=g, device="cuda").half()
    w = (torch.rand(4096, generator=g, device="cuda") + 0.5).half()
    want_x = x + r
    want_y = ops.rmsnorm(want_x, w, 1e-5)
    xs = x.clone()
    got_y = ops.add_rmsnorm(xs, r, w, 1e-5)
    assert torch.equal(xs, want_x)          # the fp16 sum, in place
    assert torch.equal(got_y, want_y)       # same reduction as the plain norm kernel


@pytest.mark.parametrize("hq,hkv", [(64, 8), (32, 4), (8, 8), (16, 8), (32, 8)])
@pytest.mark.parametrize("B,max_len,p", [(1, 512, 0), (1, 512, 5), (2, 512, 63), (1, 512, 64), (3, 512, 383), (1, 512, 511),
                                         (2, 128, 100), (1, 64, 40), (1, 1024, 700), (1, 4096, 4095), (1, 200, 199)])
def test_decode_attention_matches_an_fp32_reference(hq, hkv, B, max_len, p):
    """One query per row over the keys 0..p of the static cache, against softmax(q k^T / sqrt(d)) v in fp32."""
    hd = 128
    g = torch.Generator(device="cuda").manual_seed(hq * 1000 + max_len + p)
    qkv = torch.randn(B, 1, hq + 2 * hkv, hd, generator=g, device="cuda").half()
    kc = torch.randn(B, hkv, max_len, hd, generator=g, device="cuda").half()
    vc = torch.randn(B, hkv, max_len, hd, generator=g, device="cuda").half()
    # positions past p hold values that must not leak into the result
    kc[:, :, p + 1 :] = 1000.0
    vc[:, :, p + 1 :] = 1000.0
    pos = torch.tensor([p], dtype=torch.int64, device="cuda")
    assert ops.decode_attention_supported(hq, hkv, hd, max_len)
    out = ops.decode_attention(qkv, pos, kc, vc, hq, hkv)
    q = qkv[:, 0, :hq].float()                                       # [B, hq, hd]
    G = hq // hkv
    k = kc[:, :, : p + 1].float().repeat_interleave(G, dim=1)        # [B, hq, n, hd]
    v = vc[:, :, : p + 1].float().repeat_interleave(G, dim=1)
    s = torch.einsum("bhd,bhnd->bhn", q, k) / hd ** 0.5
    ref = torch.einsum("bhn,bhnd->bhd", torch.softmax(s, dim=-1), v).reshape(B, hq * hd)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-3 * max(1.0, ref.abs().max().item()), err


def test_decode_attention_rejects_unsupported_shapes():
    assert not ops.decode_attention_supported(64, 8, 64, 512)      # head dimension
    assert not ops.decode_attention_supported(48, 8, 128, 512)     # six query heads per key/value head
    assert not ops.decode_attention_supported(64, 8, 128, 1 << 15)


def test_decode_step_with_native_attention_matches_torch_ops():
    """A prefill, then single-token steps: the native attention (head dimension 128, four query heads
    per key/value head) against the framework's masked attention over the whole cache."""
    cfg = DecoderConfig(layers=2, d_model=1024, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64)
    assert cfg.head_dim == 128
    a = QuantDecoder(cfg, device="cuda", seed=5, batch=2, native_ops=True)
    b = QuantDecoder(cfg, device="cuda", seed=5, batch=2, native_ops=False)
    for m in (a, b):
        for blk in m.blocks:
            for l in (blk.qkv, blk.o, blk.gate_up, blk.down):
                l.s.mul_(20.0)
    tokens = torch.randint(0, cfg.vocab, (2, 9), device="cuda")
    with torch.no_grad():
        a(tokens, torch.arange(9, device="cuda"))
        b(tokens, torch.arange(9, device="cuda"))
        for step in range(3):
            tok = torch.randint(0, cfg.vocab, (2, 1), device="cuda")
            pos = torch.tensor([9 + step], device="cuda")
            ya, yb = a(tok, pos).float(), b(tok, pos).float()
            assert torch.isfinite(ya).all()
            assert (ya - yb).abs().max() <= 5e-3 * yb.abs().max()


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K,GS,bits", [(384, 1024, 128, 4), (4096, 11008, 128, 4), (200, 2048, 64, 4), (512, 3584, 128, 8), (256, 1024, -1, 2)])
def test_down_projection_with_fused_silu_mul(M, N, K, GS, bits):
    """silu(gate) * up combined inside the GEMV's activation staging: bit-identical to the element-wise
    kernel followed by the plain forward, and within the parity bar of the oracle applied to the
    fp16 activation the reference's serving stack would compute."""
    import numpy as np

    from oracle import qf_oracle as O
    from qfactory import QLinear, _native, ops

    _, q, s, z = O.make_case(M, N, K, bits, GS, False, seed=M + N)
    if GS == -1:
        layer = QLinear.init(M, K, N, bits, q.cuda(), layout="fragment")
    else:
        layer = QLinear.init(M, K, N, bits, q.cuda(), GS, s.cuda(), z.cuda(), layout="fragment")
    g = torch.Generator().manual_seed(M * 7 + K)
    gu = torch.randn(M, 2 * K, generator=g).half()
    assert layer.silu_mul_supported(M)
    y = layer.forward_silu_mul(gu.cuda())
    assert _native.last_launch()["kernel"] == 3
    act = ops.silu_mul(gu.cuda())
    assert torch.equal(y, layer(act))
    # the oracle on the activation as torch computes it (fp32 silu rounded to fp16, fp16 product)
    act_ref = torch.nn.functional.silu(gu[:, :K].float()).half() * gu[:, K:]
    _, yex = O.reference_forward(act_ref, q, s, z, bits)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= 1e-2 * np.abs(yex).max()


def test_fused_silu_mul_falls_back_above_16_rows_and_on_tile_layers():
    from oracle import qf_oracle as O
    from qfactory import QLinear, ops

    M, N, K = 20, 256, 1024
    _, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=3)
    gu = torch.randn(M, 2 * K, generator=torch.Generator().manual_seed(1)).half().cuda()
    for lay, rows in (("fragment", 20), ("tile", 4)):
        layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout=lay)
        assert not layer.silu_mul_supported(rows)
        y = layer.forward_silu_mul(gu[:rows])
        assert torch.equal(y, layer(ops.silu_mul(gu[:rows].contiguous())))


@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 2), (64, 8), (8, 1)])
@pytest.mark.parametrize("B,max_len,p", [(1, 512, 0), (1, 512, 7), (2, 512, 130), (3, 512, 383), (1, 4096, 4095), (2, 2048, 1000)])
def test_fused_rope_attention_equals_the_two_separate_launches(hq, hkv, B, max_len, p):
    """Rotary embedding + cache write + attention of one new token in ONE launch: the output, the
    cache contents at the new position and everything else are bit-identical to `rope_cache`
    followed by `decode_attention` (whose results are checked against torch elsewhere)."""
    hd = 128
    g = torch.Generator(device="cuda").manual_seed(hq * 100 + hkv * 10 + p)
    qkv = torch.randn(B, 1, hq + 2 * hkv, hd, generator=g, device="cuda").half()
    kc = torch.randn(B, hkv, max_len, hd, generator=g, device="cuda").half()
    vc = torch.randn(B, hkv, max_len, hd, generator=g, device="cuda").half()
    kc[:, :, p:] = 1000.0     # position p itself must come from the new token, later ones must not leak in
    vc[:, :, p:] = 1000.0
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().half(), ang.sin().half()
    pos = torch.tensor([p], dtype=torch.int64, device="cuda")
    # two launches on copies
    qkv_a, kc_a, vc_a = qkv.clone(), kc.clone(), vc.clone()
    ops.rope_cache(qkv_a, cos, sin, pos, kc_a, vc_a, hq, hkv)
    want = ops.decode_attention(qkv_a, pos, kc_a, vc_a, hq, hkv)
    # one launch
    qkv_b, kc_b, vc_b = qkv.clone(), kc.clone(), vc.clone()
    got = ops.decode_attention_rope(qkv_b, cos, sin, pos, kc_b, vc_b, hq, hkv)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert torch.equal(kc_b, kc_a) and torch.equal(vc_b, vc_a)     # the new key / value landed, nothing else changed
    assert torch.equal(qkv_b, qkv)                                  # the fused kernel leaves qkv alone


def test_decoder_with_and_without_fused_rope_gives_the_same_logits():
    cfg = DecoderConfig(layers=2, d_model=1024, n_heads=8, n_kv_heads=2, d_ff=1024, vocab=1000, max_len=64, scale_boost=40.0)
    a = QuantDecoder(cfg, device="cuda", seed=6, batch=2, weights="seeded")
    b = QuantDecoder(cfg, device="cuda", seed=6, batch=2, weights="seeded")
    b.fuse_rope = False
    tokens = torch.randint(0, cfg.vocab, (2, 9), device="cuda")
    with torch.no_grad():
        assert torch.equal(a(tokens, torch.arange(9, device="cuda")), b(tokens, torch.arange(9, device="cuda")))
        for step in range(3):
            tok = torch.randint(0, cfg.vocab, (2, 1), device="cuda")
            pos = torch.tensor([9 + step], device="cuda")
            assert torch.equal(a(tok, pos), b(tok, pos))
