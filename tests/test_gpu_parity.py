"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bar: integer work (packed bytes, unpacked codes, dequantised fp16 bit patterns) is
bit-exact; outputs are within max-abs <= 1e-2 * ||y||_inf of the oracle's
dequantize-then-matmul (fp16 operands, exact contraction)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import QLinear, _native, layout
from qfactory.convert import convert_params

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max-abs error allowed, as a fraction of ||y||_inf


def _layer(N, K, bits, GS, sym, seed=0, M=1, layout_kind="tile"):
    x, q, s, z = O.make_case(M, N, K, bits, GS, sym, seed)
    if GS == -1:
        layer = QLinear.init(M, K, N, bits, q.cuda(), layout=layout_kind)
    else:
        layer = QLinear.init(M, K, N, bits, q.cuda(), GS, s.cuda(), None if z is None else z.cuda(), layout=layout_kind)
    return layer, x, q, s, z


def _check_output(y_gpu, x, q, s, z, bits):
    y16, yex = O.reference_forward(x, q, s, z, bits)
    got = y_gpu.float().cpu().numpy().astype(np.float64)
    scale = np.abs(yex).max()
    err = np.abs(got - yex).max()
    assert err <= TOL * scale, f"max-abs {err} > {TOL} * {scale}"
    # and the fp16 CPU matmul of the reference test path sits inside the same band
    assert np.abs(y16.double().numpy() - yex).max() <= TOL * scale
    return err / scale


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("N", [64, 128, 300])
def test_device_packer_matches_host_packer(bits, N):
    K, GS = 512, 128
    _, q, s, z = O.make_case(1, N, K, bits, GS, False, seed=7)
    args = {"K": K, "N": N, "NBITS": bits, "GS": GS}
    wc, sc, zc = convert_params(args, (q, s, z))
    wg, sg, zg = convert_params(args, (q.cuda(), s.cuda(), z.cuda()))
    assert torch.equal(wg.cpu(), wc) and torch.equal(sg.cpu().view(torch.int16), sc.view(torch.int16))
    assert torch.equal(zg.cpu(), zc)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("N,K", [(128, 256), (200, 512), (1, 128), (384, 1024)])
def test_unpacked_codes_bit_exact(bits, N, K):
    layer, x, q, s, z = _layer(N, K, bits, 128, False, seed=bits + N)
    assert torch.equal(layer.unpack_codes().cpu(), q)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("sym", [False, True])
def test_dequantised_weight_bit_exact(bits, sym):
    N, K, GS = 200, 512, 128
    layer, x, q, s, z = _layer(N, K, bits, GS, sym, seed=11 + bits)
    ze = O.symmetric_zero(bits) if sym else O.effective_zero(z.numpy(), bits)
    want = O.dequant_effective(q, s, ze)
    got = layer.dequantize().cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


KERNEL_FLAGS = {"simt": _native.FLAG_FORCE_SIMT, "tensor": _native.FLAG_FORCE_TENSOR, "auto": 0}


@pytest.mark.parametrize("kernel", ["simt", "tensor"])
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 8, 16, 17])
def test_forward_small_shapes(bits, M, kernel):
    N, K, GS = 328, 1024, 128
    layer, x, q, s, z = _layer(N, K, bits, GS, False, seed=100 * bits + M, M=M)
    layer.flags = KERNEL_FLAGS[kernel]
    y = layer(x.cuda())
    assert _native.last_launch()["kernel"] == (1 if kernel == "simt" else 2)
    assert y.shape == (M, N) and y.dtype == torch.float16
    _check_output(y, x, q, s, z, bits)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("GS,sym", [(128, True), (64, False), (256, False), (-1, False)])
@pytest.mark.parametrize("kernel", ["simt", "tensor"])
def test_forward_modes(bits, GS, sym, kernel):
    if bits == 3 and GS == 64:
        GS = 128
    N, K = 256, 2048
    layer, x, q, s, z = _layer(N, K, bits, GS, sym, seed=bits * 7 + (GS % 97), M=2)
    layer.flags = KERNEL_FLAGS[kernel]
    y = layer(x.cuda())
    _check_output(y, x, q, s, z, bits)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_forward_on_golden_fixture(golden_dir, bits):
    f = np.load(os.path.join(golden_dir, f"dequant_b{bits}.npz"))
    K, N, GS, M = int(f["K"]), int(f["N"]), int(f["GS"]), int(f["M"])
    q, s, z = torch.from_numpy(f["q"]), torch.from_numpy(f["s"]), torch.from_numpy(f["z"])
    layer = QLinear.init(M, K, N, bits, q.cuda(), GS, s.cuda(), z.cuda(), layout="tile")
    y = layer(torch.from_numpy(f["x"]).cuda()).float().cpu().numpy()
    ref = f["y"].astype(np.float32)  # produced by the reference's own dequant + fp16 matmul
    assert np.abs(y - ref).max() <= TOL * np.abs(ref).max()
    # the dequantised weight equals the reference helper's output bit for bit (no clamp in play here)
    assert np.array_equal(layer.dequantize().cpu().numpy().view(np.uint16), f["wdq"].view(np.uint16))
    g = QLinear.init(M, K, N, bits, q.cuda(), layout="tile")
    yg = g(torch.from_numpy(f["x"]).cuda()).float().cpu().numpy()
    refg = f["y_groupless"].astype(np.float32)
    assert np.abs(yg - refg).max() <= TOL * np.abs(refg).max()


def test_clamped_top_zero_follows_packer_semantics():
    # z == 2^b - 1 is stored as 2^b - 1 (not 2^b): kernel == packer semantics, one step off the unclamped helper
    bits, N, K, GS = 4, 128, 256, 128
    x, q, s, z = O.make_case(1, N, K, bits, GS, False, seed=3)
    z[:] = 15
    layer = QLinear.init(1, K, N, bits, q.cuda(), GS, s.cuda(), z.cuda(), layout="tile")
    want = O.dequant_effective(q, s, np.full((K // GS, N), 15, dtype=np.int32))
    assert torch.equal(layer.dequantize().cpu().view(torch.int16), want.view(torch.int16))


SHAPES_7B = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]
LAYOUTS = ["tile", "fragment"]


def _expected_kernel(layout_kind, M):
    """Kernel id a fragment-layout layer must launch: the mma.sync GEMV up to 16 rows, the
    tcgen05 kernel above (None: tile-layout layers choose between kernels 1 and 2 by size)."""
    if layout_kind != "fragment":
        return None
    return 3 if M <= 16 else 2


@pytest.mark.parametrize("layout_kind", LAYOUTS)
@pytest.mark.parametrize("N,K", SHAPES_7B)
@pytest.mark.parametrize("M", [1, 4, 16])
def test_llama7b_layer_shapes_against_oracle(N, K, M, layout_kind):
    """Every case of the Llama-7B layer sweep (reference: tests/acc_gptq.py:40-72 runs each
    shape x M x bits against dequantize-then-matmul), on the layout the benchmark launches too."""
    layer, x, q, s, z = _layer(N, K, 4, 128, False, seed=0, M=M, layout_kind=layout_kind)
    y = layer(x.cuda())
    want = _expected_kernel(layout_kind, M)
    if want is not None:
        assert _native.last_launch()["kernel"] == want
    rel = _check_output(y, x, q, s, z, 4)
    assert rel < TOL


@pytest.mark.parametrize("layout_kind", LAYOUTS)
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("sym", [False, True])
def test_bit_width_sweep_8192(bits, sym, layout_kind):
    N = K = 8192
    layer, x, q, s, z = _layer(N, K, bits, 128, sym, seed=0, M=1, layout_kind=layout_kind)
    y = layer(x.cuda())
    want = _expected_kernel(layout_kind, 1)
    if want is not None:
        assert _native.last_launch()["kernel"] == want
    _check_output(y, x, q, s, z, bits)


def _random_packed_layer(N, K, bits, GS, M, layout_kind, seed):
    """A full-size layer of random packed bytes (any byte pattern is a valid packing), its
    activations, and the codes / scales / zeros of a few sampled output rows recovered by the
    torch unpackers, for a sampled oracle check where the whole oracle would take minutes."""
    g = torch.Generator().manual_seed(seed)
    layer = QLinear.empty(M, K, N, bits, GS, sym=False, layout=layout_kind)
    layer.w.copy_(torch.randint(-128, 128, layer.w.shape, generator=g, dtype=torch.int8))
    layer.s.copy_((torch.rand(layer.s.shape, generator=g) * 0.018 + 0.002).half())
    layer.z.copy_(torch.randint(0, 1 << bits, layer.z.shape, generator=g, dtype=torch.int8))
    x = torch.randn(M, K, generator=g).half()
    return layer, x


def _sampled_oracle(layer, x, rows):
    N = layer.out_features
    q = layer.unpack_codes()[:, rows].cpu()
    frag = layer.packed_layout == layout.LAYOUT_FRAGMENT
    s = (layout.unpack_scale_fragment if frag else layout.unpack_scale)(layer.s.cpu(), N)[:, rows]
    ze = (layout.unpack_zero_fragment if frag else layout.unpack_zero)(layer.z.cpu(), N)[:, rows].numpy()
    return O.qlinear_exact(x, O.dequant_effective(q, s, ze))


@pytest.mark.parametrize("layout_kind", LAYOUTS)
@pytest.mark.parametrize("N,K", [(28672, 8192), (8192, 28672)])
@pytest.mark.parametrize("M", [1, 8, 16, 32, 64, 128, 256, 1024])
def test_llama70b_mlp_shapes_sampled_rows(N, K, M, layout_kind):
    """Batch sweep on both Llama-70B MLP shapes at full size, built-in kernel choice: sampled
    output rows against the oracle, crossing from the GEMV kernels to the tcgen05 kernel."""
    layer, x = _random_packed_layer(N, K, 4, 128, M, layout_kind, seed=M + N)
    y = layer(x.cuda())
    want_kernel = _expected_kernel(layout_kind, M)
    if want_kernel is not None:
        assert _native.last_launch()["kernel"] == want_kernel
    rows = torch.tensor([0, 1, 127, 128, N // 2 + 5, N - 1])
    want = _sampled_oracle(layer, x, rows)
    got = y[:, rows].float().cpu().numpy()
    assert np.isfinite(y.float().cpu().numpy()).all()
    assert np.abs(got - want).max() <= TOL * float(y.float().abs().max())


# the layer shapes of the other model families the reference sweeps (its size and bit-width figures):
# each distinct (N, K) once, at full size, on the layout the sweep runs
_FAMILY_SHAPES = [(5120, 5120), (27648, 5120), (5120, 13824), (15360, 5120), (57344, 8192), (10240, 8192),
                  (3584, 3584), (37888, 3584), (3584, 18944), (4608, 3584), (55296, 5120), (5120, 27648),
                  (7168, 5120), (59392, 8192), (8192, 29696), (16384, 16384)]


@pytest.mark.parametrize("N,K", _FAMILY_SHAPES)
@pytest.mark.parametrize("M", [1, 16])
def test_other_family_shapes_sampled_rows(N, K, M):
    """K = 3584, 13824, 18944, 27648, 29696 are not powers of two (28 ... 232 batches of 128 k): the
    split-K ranges are uneven there.  Sampled output rows against the oracle, fragment layout."""
    layer, x = _random_packed_layer(N, K, 4, 128, M, "fragment", seed=N + K + M)
    y = layer(x.cuda())
    assert _native.last_launch()["kernel"] == 3
    rows = torch.tensor([0, 1, 127, 128, N // 2 + 5, N - 1])
    want = _sampled_oracle(layer, x, rows)
    got = y[:, rows].float().cpu().numpy()
    assert np.isfinite(y.float().cpu().numpy()).all()
    assert np.abs(got - want).max() <= TOL * float(y.float().abs().max())


@pytest.mark.parametrize("layout_kind", LAYOUTS)
@pytest.mark.parametrize("N,K", [(28672, 8192), (8192, 28672)])
def test_full_size_properties_mlp70b(N, K, layout_kind):
    # W4 g128 at full size: linearity in x, determinism, and a sampled oracle check
    layer, x1 = _random_packed_layer(N, K, 4, 128, 1, layout_kind, seed=0)
    g = torch.Generator().manual_seed(1)
    x2 = torch.randn(1, K, generator=g).half().cuda()
    x1 = x1.cuda()
    y1, y2 = layer(x1).float(), layer(x2).float()
    y12 = layer((x1.float() + x2.float()).half()).float()
    scale = y12.abs().max()
    assert (y12 - (y1 + y2)).abs().max() <= 2 * TOL * scale
    assert torch.equal(layer(x1), layer(x1))  # split-K reduction order is fixed
    rows = torch.tensor([0, 1, 127, 128, 5000, N - 1])
    want = _sampled_oracle(layer, x1.cpu(), rows)
    got = layer(x1)[:, rows].float().cpu().numpy()
    assert np.abs(got - want).max() <= TOL * float(scale)


@pytest.mark.parametrize("split,kways", [(1, 1), (2, 2), (5, 1), (16, 2), (64, 1), (1000, 2)])
def test_split_k_settings_agree(split, kways):
    N, K, bits, GS = 384, 4096, 4, 128
    layer, x, q, s, z = _layer(N, K, bits, GS, False, seed=9, M=3)
    layer.flags = _native.FLAG_FORCE_SIMT
    L = _native.lib()
    try:
        L.qfb_set_gemv_tuning(split, kways)
        y = layer(x.cuda())
        info = _native.last_launch()
    finally:
        L.qfb_set_gemv_tuning(0, 0)
    assert info["kernel"] == 1 and info["grid_y"] == 3
    _check_output(y, x, q, s, z, bits)


def test_repeated_calls_reuse_the_workspace():
    layer, x, q, s, z = _layer(512, 2048, 4, 128, False, seed=2, M=1)
    xs = x.cuda()
    ys = [layer(xs).clone() for _ in range(5)]
    for y in ys[1:]:
        assert torch.equal(y, ys[0])


def test_leading_dimensions_and_out_argument():
    layer, x, q, s, z = _layer(256, 512, 4, 128, False, seed=4, M=6)
    xs = x.cuda().view(2, 3, 512)
    y = layer(xs)
    assert y.shape == (2, 3, 256)
    out = torch.empty(6, 256, dtype=torch.float16, device="cuda")
    y2 = layer(x.cuda(), out=out)
    assert y2.data_ptr() == out.data_ptr() and torch.equal(y.view(6, 256), out)


def test_host_buffer_entry_matches_device_entry():
    layer, x, q, s, z = _layer(640, 1024, 4, 128, False, seed=5, M=4)
    xh = x.pin_memory()
    yh = torch.empty(4, 640, dtype=torch.float16).pin_memory()
    layer.forward_host(xh, yh)
    assert torch.equal(yh, layer(x.cuda()).cpu())
    # queued form: nothing is waited for until the caller synchronises the stream
    yq = torch.zeros(4, 640, dtype=torch.float16).pin_memory()
    layer.forward_host(xh, yq, sync=False)
    torch.cuda.current_stream().synchronize()
    assert torch.equal(yq, yh)


def test_pdl_flag_gives_identical_results():
    layer, x, q, s, z = _layer(1024, 4096, 4, 128, False, seed=6, M=1)
    xs = x.cuda()
    y0 = layer(xs).clone()
    layer.flags = _native.FLAG_PDL
    ys = [layer(xs).clone() for _ in range(4)]
    torch.cuda.synchronize()
    for y in ys:
        assert torch.equal(y, y0)


def test_status_codes_on_device():
    L = _native.lib()
    layer, x, q, s, z = _layer(128, 4096, 4, 128, False, seed=1, M=1)
    layer.flags = _native.FLAG_FORCE_SIMT
    xs = x.cuda()
    y = layer(xs)
    d = layer._desc
    # split-K needs a workspace
    st = L.qfb_linear_forward(ctypes.byref(d), xs.data_ptr(), 1, y.data_ptr(), None, 0, _native.FLAG_FORCE_SIMT, None)
    assert st == 5
    torch.cuda.synchronize()


def test_state_dict_round_trip():
    layer, x, q, s, z = _layer(256, 512, 4, 128, False, seed=8, M=1)
    sd = {k: v.cpu() for k, v in layer.state_dict().items()}
    other = QLinear.empty(1, 512, 256, 4, 128, sym=False, layout="tile")
    other.load_state_dict(sd)
    assert torch.equal(other(x.cuda()), layer(x.cuda()))


def test_from_float_front_end():
    g = torch.Generator().manual_seed(12)
    w = torch.randn(512, 256, generator=g).half()
    x = torch.randn(2, 512, generator=g).half()
    layer = QLinear.from_float(w.cuda(), 4, 128, layout="tile")
    q, s, z = O.asymmetric_quant(w, 128, 4)
    _check_output(layer(x.cuda()), x, q, s, z, 4)
    # the reference's own criterion (tests/acc_gptq.py:61-62): MSE against dequantize-then-matmul < 0.1
    y = layer(x.cuda()).float().cpu()
    yq = (x @ O.dequant_unclamped(q, s, z)).float()
    assert round(((y - yq) ** 2).mean().item(), 4) < 0.1
