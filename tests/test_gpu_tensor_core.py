"""GPU parity tests of the tcgen05 tensor-core kernel, forced through the C ABI, against the
CPU oracle: every batch-tile width, both accumulation modes (per-group accumulators with
fp32 post-scaling, and scaling in the decode), split-K, ragged edges, and the status word
that bounded waits would raise."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import QLinear, _native

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _run(M, N, K, bits, GS, sym, seed, flags=_native.FLAG_FORCE_TENSOR):
    x, q, s, z = O.make_case(M, N, K, bits, GS, sym, seed)
    if GS == -1:
        layer = QLinear.init(M, K, N, bits, q.cuda(), layout="tile")
    else:
        layer = QLinear.init(M, K, N, bits, q.cuda(), GS, s.cuda(), None if z is None else z.cuda(), layout="tile")
    layer.flags = flags
    y = layer(x.cuda())
    torch.cuda.synchronize()
    info = _native.last_launch()
    st = ctypes.c_uint(0)
    rc = _native.lib().qfb_read_status(layer._ws.data_ptr(), None, ctypes.byref(st))
    assert rc == 0 and st.value == 0, "a bounded wait ran out on the device"
    _, yex = O.reference_forward(x, q, s, z, bits)
    err = np.abs(y.float().cpu().numpy() - yex).max()
    scale = np.abs(yex).max()
    assert err <= TOL * scale, f"max-abs {err} > {TOL} * {scale}"
    return info, layer, x


@pytest.mark.parametrize("M", [1, 5, 16, 17, 32, 33, 64, 65, 100, 128, 129, 256, 257, 300, 600])
def test_every_batch_tile_width(M):
    info, _, _ = _run(M, 384, 2048, 4, 128, False, seed=M)
    assert info["kernel"] == 2


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("M", [3, 48, 200])
@pytest.mark.parametrize("sym", [False, True])
def test_bit_widths_in_both_accumulation_modes(bits, M, sym):
    _run(M, 256, 1024, bits, 128, sym, seed=bits * 10 + M)


@pytest.mark.parametrize("GS", [64, 128, 256, 512, -1])
@pytest.mark.parametrize("M", [4, 40, 130])
def test_group_sizes(GS, M):
    _run(M, 256, 2048, 4, GS, False, seed=GS % 101 + M)


@pytest.mark.parametrize("N", [1, 100, 128, 129, 1000])
def test_ragged_output_rows(N):
    _run(7, N, 1024, 4, 128, False, seed=N)
    _run(150, N, 1024, 4, 128, False, seed=N + 1)


@pytest.mark.parametrize("K", [128, 256, 384, 1152, 11008])
def test_k_extents_and_split_k(K):
    info, _, _ = _run(2, 256, K, 4, 128, False, seed=K % 97)
    if K >= 1024:
        assert info["grid_y"] > 1  # K was split across CTAs
    _run(70, 256, K, 8, 128, False, seed=K % 89)


def test_tensor_kernel_falls_back_when_k_is_not_a_stage_multiple():
    # K = 192 is a multiple of 64 but not of 128: the tensor path does not apply
    x, q, s, z = O.make_case(4, 128, 192, 4, 64, False, 3)
    layer = QLinear.init(4, 192, 128, 4, q.cuda(), 64, s.cuda(), z.cuda(), layout="tile")
    layer.flags = _native.FLAG_FORCE_TENSOR
    y = layer(x.cuda())
    assert _native.last_launch()["kernel"] == 1
    _, yex = O.reference_forward(x, q, s, z, 4)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()


def test_deterministic_and_workspace_reuse():
    _, layer, x = _run(8, 512, 4096, 4, 128, False, seed=1)
    xs = x.cuda()
    ys = [layer(xs).clone() for _ in range(6)]
    for y in ys[1:]:
        assert torch.equal(y, ys[0])


def test_pdl_launches_give_identical_results():
    _, layer, x = _run(4, 1024, 4096, 4, 128, False, seed=2)
    xs = x.cuda()
    y0 = layer(xs).clone()
    layer.flags = _native.FLAG_FORCE_TENSOR | _native.FLAG_PDL
    ys = [layer(xs).clone() for _ in range(4)]
    torch.cuda.synchronize()
    for y in ys:
        assert torch.equal(y, y0)


def test_simt_and_tensor_kernels_agree():
    x, q, s, z = O.make_case(6, 640, 2048, 4, 128, False, 5)
    layer = QLinear.init(6, 2048, 640, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="tile")
    layer.flags = _native.FLAG_FORCE_SIMT
    a = layer(x.cuda()).float()
    layer.flags = _native.FLAG_FORCE_TENSOR
    b = layer(x.cuda()).float()
    assert (a - b).abs().max() <= 2e-3 * a.abs().max()


@pytest.mark.parametrize("M", [1, 16, 64, 128, 1024])
def test_llama70b_mlp_shape_sampled_rows(M):
    # (28672, 8192) W4 g128 at full size: sampled output rows against the oracle
    N, K, bits, GS = 28672, 8192, 4, 128
    g = torch.Generator().manual_seed(M)
    layer = QLinear.empty(M, K, N, bits, GS, sym=False, layout="tile")
    layer.w.copy_(torch.randint(-128, 128, layer.w.shape, generator=g, dtype=torch.int8))
    layer.s.copy_((torch.rand(layer.s.shape, generator=g) * 0.018 + 0.002).half())
    layer.z.copy_(torch.randint(0, 16, layer.z.shape, generator=g, dtype=torch.int8))
    layer.flags = _native.FLAG_FORCE_TENSOR
    x = torch.randn(M, K, generator=g).half()
    y = layer(x.cuda())
    from qfactory import layout

    rows = torch.tensor([0, 127, 128, 4095, 14000, 28671])
    q = layer.unpack_codes()[:, rows].cpu()
    s = layout.unpack_scale(layer.s.cpu(), N)[:, rows]
    ze = layout.unpack_zero(layer.z.cpu(), N)[:, rows].numpy()
    want = O.qlinear_exact(x, O.dequant_effective(q, s, ze))
    got = y[:, rows].float().cpu().numpy()
    assert np.abs(got - want).max() <= TOL * float(y.float().abs().max())


def test_kernel_selection_rule():
    L = _native.lib()
    assert L.qfb_select_kernel(1, 4096, 4096, 4, 0) == 1          # small weight, one row: CUDA cores
    assert L.qfb_select_kernel(1, 28672, 8192, 4, 0) == 2         # large weight: tensor pipeline
    assert L.qfb_select_kernel(4, 4096, 4096, 4, 0) == 2
    assert L.qfb_select_kernel(4, 4096, 4096, 4, _native.FLAG_FORCE_SIMT) == 1
    assert L.qfb_select_kernel(4, 4096, 4160, 4, 0) == 1          # K not a multiple of 128


@pytest.mark.parametrize("M,GS,bits", [(40, 128, 4), (64, 64, 4), (130, 128, 4), (300, 256, 8), (200, 128, 2), (90, -1, 4), (150, 128, 3)])
def test_one_and_two_decode_groups_give_identical_results(M, GS, bits):
    """Where the scale is applied in the decode the kernel runs two decode groups on alternate
    stages (768 threads); one group (512 threads) must give the same bits."""
    L = _native.lib()
    try:
        L.qfb_set_tensor_decode_groups(2)
        info2, layer, x = _run(M, 384, 2048, bits, GS, False, seed=900 + M)
        xs = x.cuda()
        y2 = layer(xs).clone()
        L.qfb_set_tensor_decode_groups(1)
        y1 = layer(xs).clone()
        info1 = _native.last_launch()
        torch.cuda.synchronize()
    finally:
        L.qfb_set_tensor_decode_groups(0)
    assert torch.equal(y1, y2)
    # 16- and 32-wide batch tiles with per-stage accumulators always run one group
    if info2["block"] == 768:
        assert info1["block"] == 512


@pytest.mark.parametrize("M,bits,GS", [(130, 4, 128), (300, 4, 128), (257, 8, 64), (100, 2, -1)])
@pytest.mark.parametrize("layout_kind", ["tile", "fragment"])
def test_tail_split_of_wide_batches_agrees_with_the_plain_grid(M, bits, GS, layout_kind):
    """Above 64 rows the units of a launch's last, partly filled wave are cut along K (2..4 ranges,
    fp32 partials summed in range order by the last CTA to arrive).  Forced here on every unit and
    compared with the oracle and with the uncut launch."""
    L = _native.lib()
    N, K = 384, 4096
    x, q, s, z = O.make_case(M, N, K, bits, GS, False, seed=700 + M)
    if GS == -1:
        layer = QLinear.init(M, K, N, bits, q.cuda(), layout=layout_kind)
    else:
        layer = QLinear.init(M, K, N, bits, q.cuda(), GS, s.cuda(), z.cuda(), layout=layout_kind)
    layer.flags = _native.FLAG_FORCE_TENSOR
    layer._prepare()
    # cutting EVERY unit in four needs more partial-sum space than the built-in plan ever asks for
    layer._ws = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    layer._ws_bytes = layer._ws.numel()
    xs = x.cuda()
    _, yex = O.reference_forward(x, q, s, z, bits)
    outs = {}
    try:
        for split in (1, 2, 3, 4):
            L.qfb_set_tensor_split(split)
            y = layer(xs).clone()
            info = _native.last_launch()
            assert info["kernel"] == 2 and info["grid_y"] == split
            assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()
            assert torch.equal(y, layer(xs))   # fixed summation order: identical between runs
            outs[split] = y.float()
    finally:
        L.qfb_set_tensor_split(0)
    st = ctypes.c_uint(0)
    assert L.qfb_read_status(layer._ws.data_ptr(), None, ctypes.byref(st)) == 0 and st.value == 0
    for split in (2, 3, 4):
        assert (outs[split] - outs[1]).abs().max() <= 2e-3 * outs[1].abs().max()


def test_wide_tile_with_k_split_when_the_row_tiles_leave_most_sms_idle():
    # 16 row tiles at 128 rows: a 128-column batch tile cut in K ranges instead of two 64-column tiles
    M, N, K = 128, 2048, 8192
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=41)
    _, yex = O.reference_forward(x, q, s, z, 4)
    big = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda())       # workspace sized for 128 rows
    y = big(x.cuda())
    info = _native.last_launch()
    assert info["kernel"] == 2 and info["grid_y"] > 1 and info["smem"] == 128   # (the last field reports the batch tile)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()
    assert torch.equal(y, big(x.cuda()))
    # a workspace too small for the partial sums means the plain grid, not an error
    big._ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    big._ws_bytes = 4096
    y2 = big(x.cuda())
    assert _native.last_launch()["grid_y"] == 1
    assert np.abs(y2.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()
