"""The allocation-free entry point, for hosts that may not call cudaMalloc (their device
memory is owned by another component, or they run inside a fixed schedule or a sandbox).

Collected last on purpose.  It drives `qfb_gemv_forward_static` directly through the C ABI,
twice in a row on the same layer (the second call sees the scratch contents the first one
left behind), and compares with the regular workspace-based entry point and with the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import QLinear, _native

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max-abs error as a fraction of ||y||_inf, the bar of the other parity tests


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (5, 1000, 2048), (11, 384, 1024)])
def test_static_scratch_entry_matches_regular_entry(M, N, K):
    L = _native.lib()
    x, q, s, z = O.make_case(M, N, K, 4, 128, False, seed=31 + M)
    layer = QLinear.init(M, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="tile")
    xs = x.cuda()
    want = layer(xs).float()  # regular entry point, caller-provided workspace
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):
        y = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        st = L.qfb_gemv_forward_static(ctypes.byref(layer._desc), xs.data_ptr(), M, y.data_ptr(), 0, stream)
        assert st == 0, L.qfb_status_string(st)
        outs.append(y.float())
    torch.cuda.synchronize()
    scale = want.abs().max()
    _, yex = O.reference_forward(x, q, s, z, 4)  # the oracle's dequantize-then-matmul
    for y in outs:
        assert torch.isfinite(y).all()
        assert (y - want).abs().max() <= TOL * scale
        assert np.abs(y.cpu().numpy().astype(np.float64) - yex).max() <= TOL * np.abs(yex).max()
    assert torch.equal(outs[0], outs[1])


def test_static_scratch_rejects_oversized_requests():
    L = _native.lib()
    assert L.qfb_static_scratch_capacity() == 8 << 20
    # 131072 x 8192 at 8 rows needs far more split-K scratch than the fixed array holds
    d = _native.QfbLayer(16, 16, 16, 131072, 8192, 4, 128)
    assert L.qfb_gemv_forward_static(ctypes.byref(d), 16, 8, 16, 0, None) == 7  # QFB_ERR_TOO_LARGE
    d = _native.QfbLayer(16, 16, 16, 4096, 4000, 4, 128)
    assert L.qfb_gemv_forward_static(ctypes.byref(d), 16, 1, 16, 0, None) == 2  # bad shape
