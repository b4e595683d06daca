"""`QLinear.forward_addnorm` / `qfb_linear_addnorm_forward`: the residual add and the RMS norm fused into the
activation staging of the GEMV.  The sum written back must be bit-identical to the fp16 addition; the
result differs from norm-then-linear only by one rounding of the activations (the scalar 1 / rms is
applied to the result), so it is compared with that three-step form within a tolerance, and with the
oracle's dequantize-then-matmul on the normed activations."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import QLinear, _native, ops

pytestmark = pytest.mark.gpu
TOL = 3e-3   # of max |y|: one fp16 rounding of the activations more or less


def _norm_ref(s, w, eps):
    f = s.float()
    return (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).half() * w


@pytest.mark.parametrize("N,K", [(1024, 2048), (384, 4096), (4096, 4096), (12288, 4096), (200, 1024)])
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("with_residual", [True, False])
def test_addnorm_linear_matches_the_three_step_form(N, K, M, with_residual):
    g = torch.Generator().manual_seed(N + K + M)
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=700 + M + N)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    xs = (x.float() * 3).half().cuda()
    r = (torch.randn(M, K, generator=g) * 2).half().cuda() if with_residual else None
    w = (torch.rand(K, generator=g) + 0.5).half().cuda()
    x_out = torch.full_like(xs, float("nan"))
    y = layer.forward_addnorm(xs, r, w, 1e-5, x_out=x_out)
    assert y is not None and _native.last_launch()["kernel"] == 3
    torch.cuda.synchronize()
    want_sum = xs + r if with_residual else xs
    assert torch.equal(x_out, want_sum)
    h = _norm_ref(want_sum, w, 1e-5)
    y_ref = layer(h)
    scale = float(y_ref.float().abs().max())
    assert float((y.float() - y_ref.float()).abs().max()) <= TOL * scale
    # the oracle on the same normed activations
    _, yex = O.reference_forward(h.cpu(), q, s, z, 4)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= 1e-2 * np.abs(yex).max()
    # deterministic, and the sum may be dropped
    assert torch.equal(layer.forward_addnorm(xs, r, w, 1e-5), y)


@pytest.mark.parametrize("split,kways,mode", [(1, 1, 1), (1, 2, 1), (4, 1, 2), (8, 2, 2), (3, 1, 2)])
def test_addnorm_linear_through_forced_plans(split, kways, mode):
    """No split (one CTA per tile holds the whole row) and in-cluster splits of several sizes."""
    M, N, K = 5, 640, 4096
    L = _native.lib()
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=811)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    xs, w = x.cuda(), (torch.rand(K) + 0.5).half().cuda()
    r = torch.randn(M, K).half().cuda()
    try:
        L.qfb_set_gemv_tuning(split, kways)
        L.qfb_set_cluster_reduce(mode)
        x_out = torch.empty_like(xs)
        y = layer.forward_addnorm(xs, r, w, 1e-5, x_out=x_out)
        info = _native.last_launch()
    finally:
        L.qfb_set_gemv_tuning(0, 0)
        L.qfb_set_cluster_reduce(1)
    assert y is not None and info["grid_x"] == split
    y_ref = layer(_norm_ref(xs + r, w, 1e-5))
    assert torch.equal(x_out, xs + r)
    assert float((y.float() - y_ref.float()).abs().max()) <= TOL * float(y_ref.float().abs().max())


def test_addnorm_linear_agrees_with_the_native_norm_kernel():
    M, N, K = 2, 512, 8192
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=900)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    xs, r, w = x.cuda(), torch.randn(M, K).half().cuda(), (torch.rand(K) + 0.5).half().cuda()
    y = layer.forward_addnorm(xs, r, w, 1e-5)
    resid = xs.clone()
    h = ops.add_rmsnorm(resid, r, w, 1e-5)          # resid += r in place, h = its norm
    y_ref = layer(h)
    assert float((y.float() - y_ref.float()).abs().max()) <= TOL * float(y_ref.float().abs().max())


def test_layers_the_fused_kernel_does_not_serve_return_none():
    M, N, K = 2, 256, 1024
    for bits, lay in ((4, "tile"), (8, "fragment")):
        x, q, s, z = O.make_case(M, N, K, bits, 128, False, seed=bits)
        layer = QLinear.init(M, K, N, bits, q.cuda(), 128, s.cuda(), z.cuda(), layout=lay)
        assert layer.forward_addnorm(x.cuda(), None, torch.ones(K, dtype=torch.float16, device="cuda")) is None
    x, q, s, z = O.make_case(17, N, K, 4, 128, False, seed=1)
    layer = QLinear.init(17, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    assert layer.forward_addnorm(x.cuda(), None, torch.ones(K, dtype=torch.float16, device="cuda")) is None   # more than 16 rows
    L = _native.lib()
    xs = torch.zeros(1, K, dtype=torch.float16, device="cuda")
    layer1 = QLinear.init(1, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    layer1._prepare()
    st = L.qfb_linear_addnorm_forward(layer1._desc_ref, xs.data_ptr(), None, xs.data_ptr(), xs.data_ptr(), 1e-5, 1,
                                      torch.empty(1, N, dtype=torch.float16, device="cuda").data_ptr(), layer1._ws_ptr,
                                      layer1._ws_bytes, 0, None)
    assert st == 2     # QFB_ERR_BAD_SHAPE: the sum may not be written over an input
