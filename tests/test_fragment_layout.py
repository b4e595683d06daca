"""The tensor-core fragment layout (4-bit) and the mma.sync GEMV that reads it.

CPU part: the torch packer against the documented nibble positions, round trips, layout choice.
GPU part (marked): device packer == torch packer byte for byte, unpack / dequantise bit-exact
through the kernel's own field extraction, and the forward pass against the oracle with the same
bar as the other parity tests (max-abs <= 1e-2 * ||y||_inf)."""
import ctypes
import random

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import QLinear, _native, layout
from qfactory.convert import convert_params, unpack_params

TOL = 1e-2


def _word_index(n, k, K):
    """(word, nibble) that holds code (k, n) in the fragment layout, restated from the header."""
    tile, r = divmod(n, 128)
    wt, r = divmod(r, 64)
    rb, r = divmod(r, 16)
    h, g = divmod(r, 8)
    ks, kk = divmod(k, 16)
    t, j = divmod(kk, 4)
    nib = {(0, 0): 0, (0, 1): 4, (0, 2): 2, (0, 3): 6, (1, 0): 1, (1, 1): 5, (1, 2): 3, (1, 3): 7}[(h, j)]
    return ((((tile * 2 + wt) * (K // 16) + ks) * 32 + (g * 4 + t)) * 4 + rb), nib


def test_fragment_packer_positions_and_round_trip():
    torch.manual_seed(0)
    K, N = 256, 200
    q = torch.randint(0, 16, (K, N), dtype=torch.int32)
    w = layout.pack_weight_fragment(q)
    assert w.shape == (256, K // 2) and w.dtype == torch.int8
    assert torch.equal(layout.unpack_weight_fragment(w, N, K), q)
    words = layout._bytes_to_words(w.view(torch.uint8).reshape(-1, 4))
    rnd = random.Random(1)
    for _ in range(3000):
        n, k = rnd.randrange(N), rnd.randrange(K)
        wi, nib = _word_index(n, k, K)
        assert (int(words[wi]) >> (4 * nib)) & 15 == int(q[k, n])
    # rows beyond N are zero padding
    assert int(words[_word_index(255, 0, K)[0]]) >> (4 * _word_index(255, 0, K)[1]) & 15 == 0


def test_fragment_scale_zero_order_and_round_trip():
    K, N, GS = 512, 300, 64
    s = torch.rand(K // GS, N).half()
    z = torch.randint(0, 16, (K // GS, N), dtype=torch.int32)
    ps, pz = layout.pack_scale_fragment(s), layout.pack_zero_fragment(z, 4)
    assert torch.equal(layout.unpack_scale_fragment(ps, N), s)
    assert torch.equal(layout.unpack_zero_fragment(pz, N), layout.effective_zero(z, 4))
    flat = ps.view(-1)
    for n in (0, 9, 77, 128, 299):
        tile, r = divmod(n, 128)
        wt, r2 = divmod(r, 64)
        rb, r3 = divmod(r2, 16)
        h, g = divmod(r3, 8)
        pos = wt * 64 + g * 8 + rb * 2 + h
        for grp in (0, 5):
            assert flat[(tile * (K // GS) + grp) * 128 + pos] == s[grp, n]


def test_convert_params_layout_key_and_inverse():
    K, N, GS = 256, 130, 128
    _, q, s, z = O.make_case(1, N, K, 4, GS, False, seed=4)
    args = {"K": K, "N": N, "NBITS": 4, "GS": GS, "LAYOUT": "fragment"}
    w, ps, pz = convert_params(args, (q, s, z))
    q2, s2, z2 = unpack_params(args, (w, ps, pz))
    assert torch.equal(q2, q) and torch.equal(s2, s) and torch.equal(z2, layout.effective_zero(z, 4))
    wt, _, _ = convert_params({"K": K, "N": N, "NBITS": 4, "GS": GS}, (q, s, z))
    assert not torch.equal(w, wt)  # a different permutation of the same codes
    def nibbles(a):
        b = a.view(torch.uint8).flatten().to(torch.int16)
        return torch.sort(torch.cat([b & 15, b >> 4]))[0]

    assert torch.equal(nibbles(w), nibbles(wt))


def test_layout_choice():
    R = layout.resolve_layout
    assert R("auto", 4096, 4096, 4, 128, batch_size=1) == layout.LAYOUT_FRAGMENT
    assert R(None, 4096, 4096, 4, 128, batch_size=16) == layout.LAYOUT_FRAGMENT
    assert R("auto", 4096, 4096, 4, 128, batch_size=512) == layout.LAYOUT_FRAGMENT   # any batch size
    assert R("auto", 4096, 4096, 8, 128, batch_size=1) == layout.LAYOUT_FRAGMENT
    assert R("auto", 4096, 4096, 2, 128, batch_size=1) == layout.LAYOUT_FRAGMENT
    assert R("auto", 4096, 4096, 3, 128, batch_size=1) == layout.LAYOUT_FRAGMENT
    assert R("auto", 4096, 4160, 4, 64, batch_size=1) == layout.LAYOUT_TILE       # K % 128 != 0
    assert R("auto", 4096, 4224, 4, 192, batch_size=1) == layout.LAYOUT_TILE      # group neither 64 nor k*128
    assert R("tile", 4096, 4096, 4, 128, batch_size=1) == layout.LAYOUT_TILE
    with pytest.raises(AssertionError):
        R("fragment", 4096, 4096, 3, 64)           # 3-bit groups are multiples of 128 in both layouts
    L = _native.lib()
    assert L.qfb_layout_supported(1, 4096, 4096, 4, 128) == 1
    assert L.qfb_layout_supported(1, 4096, 4096, 8, 128) == 1
    assert L.qfb_layout_supported(1, 4096, 4096, 2, 128) == 1
    assert L.qfb_layout_supported(1, 4096, 4096, 3, 128) == 1
    assert L.qfb_layout_supported(1, 4096, 4096, 3, 64) == 0     # 3-bit groups are multiples of 128
    assert L.qfb_layout_supported(1, 4096, 4160, 4, 64) == 0
    assert L.qfb_layout_supported(0, 4096, 4160, 4, 64) == 1
    assert L.qfb_layout_supported(2, 4096, 4096, 4, 128) == 0


def test_fragment_packer_three_bits_positions():
    """3-bit: positions restated from the header, bit by bit (five fields and a spare bit per half-word)."""
    torch.manual_seed(3)
    K, N = 256, 200
    q = torch.randint(0, 8, (K, N), dtype=torch.int32)
    w = layout.pack_weight_fragment(q, 3)
    assert w.shape == (256, K * 3 // 8)
    assert torch.equal(layout.unpack_weight_fragment(w, N, K, 3), q)
    words = layout._bytes_to_words(w.view(torch.uint8).reshape(-1, 4))
    rnd = random.Random(3)
    for _ in range(4000):
        n, k = rnd.randrange(N), rnd.randrange(K)
        tile, r = divmod(n, 128)
        wt, r = divmod(r, 64)
        rb, r = divmod(r, 16)
        h, g = divmod(r, 8)
        ks, kk = divmod(k, 16)
        t, kk = divmod(kk, 4)
        lane, half, khi = g * 4 + t, (kk & 1) * 16, kk >> 1
        base = ((tile * 2 + wt) * (K // 16) + ks) * 96
        code = int(q[k, n])
        for b in range(3):
            if rb < 3:
                j, bit = rb, half + 3 * h + 9 * khi + b
            elif h == 1 and khi == 1:
                j, bit = b, half + 15
            else:
                j, bit = (2 if h else khi), half + 6 + b
            assert (int(words[base + j * 32 + lane]) >> bit) & 1 == (code >> b) & 1


@pytest.mark.parametrize("bits", [2, 8])
def test_fragment_packer_other_bit_widths(bits):
    """Positions restated from the header: word of the lane, bit inside the word, place of the word."""
    torch.manual_seed(bits)
    K, N = 256, 200
    q = torch.randint(0, 1 << bits, (K, N), dtype=torch.int32)
    w = layout.pack_weight_fragment(q, bits)
    assert w.shape == (256, K * bits // 8)
    assert torch.equal(layout.unpack_weight_fragment(w, N, K, bits), q)
    words = layout._bytes_to_words(w.view(torch.uint8).reshape(-1, 4))
    rnd = random.Random(bits)
    for _ in range(3000):
        n, k = rnd.randrange(N), rnd.randrange(K)
        tile, r = divmod(n, 128)
        wt, r = divmod(r, 64)
        rb, r = divmod(r, 16)
        h, g = divmod(r, 8)
        ks, kk = divmod(k, 16)
        t, kk = divmod(kk, 4)
        lane = g * 4 + t
        if bits == 8:
            j = 2 * rb + h
            slot, bit = (j >> 2) * 128 + lane * 4 + (j & 3), 8 * kk
        else:
            slot, bit = lane * 2 + rb // 2, (rb & 1) * 4 + h * 2 + (kk & 1) * 16 + (kk >> 1) * 8
        wi = ((tile * 2 + wt) * (K // 16) + ks) * 32 * bits + slot
        assert (int(words[wi]) >> bit) & ((1 << bits) - 1) == int(q[k, n])


# ---- GPU ---------------------------------------------------------------------------------------

def _frag_layer(M, N, K, GS, sym, seed, bits=4):
    x, q, s, z = O.make_case(M, N, K, bits, GS, sym, seed)
    if GS == -1:
        layer = QLinear.init(M, K, N, bits, q.cuda(), layout="fragment")
    else:
        layer = QLinear.init(M, K, N, bits, q.cuda(), GS, s.cuda(), None if z is None else z.cuda(), layout="fragment")
    assert layer.packed_layout == layout.LAYOUT_FRAGMENT
    return layer, x, q, s, z


def _check(y, x, q, s, z, bits=4):
    _, yex = O.reference_forward(x, q, s, z, bits)
    got = y.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert np.abs(got - yex).max() <= TOL * np.abs(yex).max()


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,GS,sym", [(128, 128, 128, False), (200, 512, 64, False), (300, 1024, 256, True), (130, 256, -1, False)])
def test_device_fragment_packer_and_inverse_bit_exact(N, K, GS, sym):
    layer, x, q, s, z = _frag_layer(1, N, K, GS, sym, seed=N + K)
    assert torch.equal(layer.w.cpu().view(torch.uint8).flatten(), layout.pack_weight_fragment(q).view(torch.uint8).flatten())
    if GS != -1:
        assert torch.equal(layer.s.cpu().view(torch.int16).flatten(), layout.pack_scale_fragment(s).view(torch.int16).flatten())
        if z is not None:
            assert torch.equal(layer.z.cpu().flatten(), layout.pack_zero_fragment(z, 4).flatten())
    assert torch.equal(layer.unpack_codes().cpu(), q)
    if GS != -1:
        ze = O.symmetric_zero(4) if sym else O.effective_zero(z.numpy(), 4)
        want = O.dequant_effective(q, s, ze)
        assert torch.equal(layer.dequantize().cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 9, 13, 16, 17, 40])
@pytest.mark.parametrize("GS,sym", [(128, False), (64, False), (256, True), (-1, False)])
def test_fragment_forward_against_oracle(M, GS, sym):
    N, K = 328, 1024
    layer, x, q, s, z = _frag_layer(M, N, K, GS, sym, seed=1000 + 17 * M + (GS % 91))
    y = layer(x.cuda())
    # up to 16 rows: the mma.sync GEMV; above: the tcgen05 kernel reading the same fragment layout
    assert _native.last_launch()["kernel"] == (3 if M <= 16 else 2)
    assert y.shape == (M, N) and y.dtype == torch.float16
    _check(y, x, q, s, z)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [17, 33, 64, 65, 130, 256, 300])
@pytest.mark.parametrize("GS,sym", [(128, False), (64, False), (256, True), (-1, False)])
def test_fragment_layer_large_batches_on_the_tcgen05_kernel(M, GS, sym):
    N, K = 384, 2048
    layer, x, q, s, z = _frag_layer(M, N, K, GS, sym, seed=2000 + M + (GS % 89))
    y = layer(x.cuda())
    assert _native.last_launch()["kernel"] == 2
    _check(y, x, q, s, z)
    st = ctypes.c_uint(0)
    assert _native.lib().qfb_read_status(layer._ws.data_ptr(), None, ctypes.byref(st)) == 0 and st.value == 0


@pytest.mark.gpu
def test_fragment_and_tile_layers_agree_on_a_large_batch():
    x, q, s, z = O.make_case(200, 640, 4096, 4, 128, False, seed=12)
    a = QLinear.init(1, 4096, 640, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    b = QLinear.init(1, 4096, 640, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="tile")
    ya, yb = a(x.cuda()), b(x.cuda())
    # same decode arithmetic ((q - z) exact, one fp16 rounding of the scale product), same MMA order
    assert torch.equal(ya, yb)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (4, 4096, 11008), (16, 12288, 4096), (1, 22016, 4096), (7, 256, 8192), (16, 128, 16384)])
def test_fragment_forward_split_k_shapes(M, N, K):
    layer, x, q, s, z = _frag_layer(M, N, K, 128, False, seed=M + N)
    xs = x.cuda()
    y = layer(xs)
    _check(y, x, q, s, z)
    y2 = layer(xs)
    assert torch.equal(y, y2)  # split order is fixed: bit-identical between runs


@pytest.mark.gpu
def test_fragment_forward_every_split_and_kway_agrees():
    L = _native.lib()
    layer, x, q, s, z = _frag_layer(3, 256, 4096, 128, False, seed=77)
    xs = x.cuda()
    try:
        for mode in (0, 2):  # K splits reduced through the workspace / inside a thread-block cluster
            L.qfb_set_cluster_reduce(mode)
            for kw in (1, 2, 4):
                for sp in (1, 2, 3, 5, 8, 32):
                    L.qfb_set_gemv_tuning(sp, kw)
                    _check(layer(xs), x, q, s, z)
    finally:
        L.qfb_set_gemv_tuning(0, 0)
        L.qfb_set_cluster_reduce(1)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 8, 16])
def test_cluster_and_workspace_reductions_agree(M):
    L = _native.lib()
    layer, x, q, s, z = _frag_layer(M, 640, 4096, 128, False, seed=5 + M)
    xs = x.cuda()
    outs = []
    try:
        for mode in (0, 2):
            L.qfb_set_cluster_reduce(mode)
            L.qfb_set_gemv_tuning(4, 2)
            outs.append(layer(xs).clone())
    finally:
        L.qfb_set_gemv_tuning(0, 0)
        L.qfb_set_cluster_reduce(1)
    _check(outs[0], x, q, s, z)
    assert torch.equal(outs[0], outs[1])  # same partials, same summation order


@pytest.mark.gpu
def test_fragment_forward_pdl_graph_and_default_layout():
    x, q, s, z = O.make_case(4, 512, 2048, 4, 128, False, seed=9)
    layer = QLinear.init(4, 2048, 512, 4, q.cuda(), 128, s.cuda(), z.cuda())  # default: auto -> fragment
    assert layer.packed_layout == layout.LAYOUT_FRAGMENT
    layer.flags = _native.FLAG_PDL
    xs = x.cuda()
    y = torch.empty(4, 512, dtype=torch.float16, device="cuda")
    layer(xs, out=y)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(3):
                layer(xs, out=y)
    y.zero_()
    g.replay()
    torch.cuda.synchronize()
    _check(y, x, q, s, z)
    other = QLinear.init(64, 2048, 512, 3, q.clamp(max=7).cuda(), 128, s.cuda(), z.clamp(max=7).cuda())  # 3-bit too
    assert other.packed_layout == layout.LAYOUT_FRAGMENT
    odd = QLinear.init(4, 2048 + 64, 512, 4, torch.cat((q, q[:64])).cuda(), 64, torch.cat((s, s[:1])).repeat_interleave(2, 0)[: (2048 + 64) // 64].cuda(),
                       torch.cat((z, z[:1])).repeat_interleave(2, 0)[: (2048 + 64) // 64].cuda())     # K % 128 != 0: tile layout
    assert odd.packed_layout == layout.LAYOUT_TILE


@pytest.mark.gpu
def test_fragment_extreme_codes_and_zeros():
    # all-15 codes with zero 0 (stored 1) and all-0 codes with zero 14 (stored 15): the largest magnitudes
    N, K, GS, M = 128, 512, 128, 2
    x = (torch.randn(M, K) * 4).half()
    s = torch.full((K // GS, N), 0.02, dtype=torch.float16)
    for code, zero in ((15, 0), (0, 14)):
        q = torch.full((K, N), code, dtype=torch.int32)
        z = torch.full((K // GS, N), zero, dtype=torch.int32)
        layer = QLinear.init(M, K, N, 4, q.cuda(), GS, s.cuda(), z.cuda(), layout="fragment")
        _check(layer(x.cuda()), x, q, s, z)


@pytest.mark.gpu
def test_fragment_forward_random_shapes_and_plans():
    """Seeded sweep over odd sizes, every group mode, forced splits / k-ways and both reductions."""
    L = _native.lib()
    rnd = random.Random(20241)
    try:
        for case in range(96):
            K = 128 * rnd.choice([1, 2, 3, 5, 8, 11, 16, 24, 32])
            N = rnd.choice([1, 7, 100, 128, 129, 255, 300, 513, 700])
            M = rnd.randint(1, 16) if case % 4 else rnd.randint(17, 70)   # every fourth case: the tcgen05 kernel
            bits = rnd.choice([2, 3, 4, 4, 8])
            gs_ok = [g for g in (64, 128, 256, 384) if K % g == 0 and not (bits == 3 and g == 64)] + [-1]
            GS = rnd.choice(gs_ok)
            sym = GS != -1 and rnd.random() < 0.3
            layer, x, q, s, z = _frag_layer(M, N, K, GS, sym, seed=5000 + case, bits=bits)
            if rnd.random() < 0.7:  # forced plan, otherwise the built-in one
                L.qfb_set_gemv_tuning(rnd.choice([1, 2, 3, 4, 6, 8, 13]), rnd.choice([1, 2, 4]))
                L.qfb_set_cluster_reduce(rnd.choice([0, 2]))
            else:
                L.qfb_set_gemv_tuning(0, 0)
                L.qfb_set_cluster_reduce(1)
            y = layer(x.cuda())
            assert _native.last_launch()["kernel"] == (3 if M <= 16 else 2)
            _check(y, x, q, s, z, bits)
    finally:
        L.qfb_set_gemv_tuning(0, 0)
        L.qfb_set_cluster_reduce(1)


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 3, 8])
@pytest.mark.parametrize("N,K,GS,sym", [(128, 128, 128, False), (200, 512, 64, False), (300, 1024, 256, True), (130, 256, -1, False)])
def test_fragment_other_bit_widths_packer_and_inverse_bit_exact(bits, N, K, GS, sym):
    if bits == 3 and GS == 64:
        GS = 128
    layer, x, q, s, z = _frag_layer(1, N, K, GS, sym, seed=N + K + bits, bits=bits)
    assert torch.equal(layer.w.cpu().view(torch.uint8).flatten(),
                       layout.pack_weight_fragment(q, bits).view(torch.uint8).flatten())
    assert torch.equal(layer.unpack_codes().cpu(), q)
    if GS != -1:
        ze = O.symmetric_zero(bits) if sym else O.effective_zero(z.numpy(), bits)
        want = O.dequant_effective(q, s, ze)
        assert torch.equal(layer.dequantize().cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 3, 8])
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 21, 40, 70, 130, 300])
@pytest.mark.parametrize("GS,sym", [(128, False), (64, False), (256, True), (-1, False)])
def test_fragment_other_bit_widths_forward(bits, M, GS, sym):
    if bits == 3 and GS == 64:
        GS = 512
    N, K = 328, 1024
    layer, x, q, s, z = _frag_layer(M, N, K, GS, sym, seed=3000 + 31 * M + bits + (GS % 83), bits=bits)
    y = layer(x.cuda())
    assert _native.last_launch()["kernel"] == (3 if M <= 16 else 2)
    _check(y, x, q, s, z, bits)


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 3, 8])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (4, 1000, 11008), (16, 2048, 4096), (1, 8192, 8192)])
def test_fragment_other_bit_widths_split_k_shapes(bits, M, N, K):
    layer, x, q, s, z = _frag_layer(M, N, K, 128, False, seed=bits + M + N, bits=bits)
    xs = x.cuda()
    y = layer(xs)
    _check(y, x, q, s, z, bits)
    assert torch.equal(y, layer(xs))
