"""The bounded device-side waits, made to run out on purpose and without any fault: a test flag
tells the kernel's first bulk-copy barrier to expect 16 bytes that never come and shortens every
wait to ~100 us.  All real copies land, nothing is in flight when the kernel leaves; it returns by
itself, raises the status word of the workspace, and the next ordinary launch is correct."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import QLinear, _native

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _status(layer):
    st = ctypes.c_uint(0)
    rc = _native.lib().qfb_read_status(layer._ws.data_ptr(), None, ctypes.byref(st))
    return rc, st.value


def _clear(layer):
    _native.check(_native.lib().qfb_workspace_init(layer._ws.data_ptr(), layer._ws_bytes,
                                                   torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("M", [1, 16])
def test_gemv_activation_barrier_wait_runs_out(M):
    x, q, s, z = O.make_case(M, 384, 2048, 4, 128, False, seed=60 + M)
    layer = QLinear.init(M, 2048, 384, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout="fragment")
    xs = x.cuda()
    want = layer(xs).clone()
    assert _status(layer) == (0, 0)
    layer.flags = _native.FLAG_TEST_STALLED_WAIT
    y = layer(xs)
    torch.cuda.synchronize()                       # the launch ended by itself
    assert _native.last_launch()["kernel"] == 3
    assert _status(layer) == (8, 1)                # QFB_ERR_DEVICE_FLAG
    assert torch.equal(y, want)                    # every copy had landed: the result is still exact
    layer.flags = 0
    _clear(layer)
    assert torch.equal(layer(xs), want) and _status(layer) == (0, 0)


@pytest.mark.parametrize("M,layout_kind", [(24, "fragment"), (100, "tile"), (200, "fragment")])
def test_tcgen05_pipeline_abandons_the_launch_and_recovers(M, layout_kind):
    """Both accumulation modes: every role of the CTA drains, tensor memory is released, the
    status word is set; the same layer then runs normally (also proving tensor memory was freed:
    a leaked allocation would leave the next CTA on that SM waiting)."""
    x, q, s, z = O.make_case(M, 256, 2048, 4, 128, False, seed=80 + M)
    layer = QLinear.init(M, 2048, 256, 4, q.cuda(), 128, s.cuda(), z.cuda(), layout=layout_kind)
    layer.flags = _native.FLAG_FORCE_TENSOR
    xs = x.cuda()
    want = layer(xs).clone()
    assert _native.last_launch()["kernel"] == 2 and _status(layer) == (0, 0)
    layer.flags = _native.FLAG_FORCE_TENSOR | _native.FLAG_TEST_STALLED_WAIT
    layer(xs)
    torch.cuda.synchronize()
    assert _status(layer) == (8, 1)
    layer.flags = _native.FLAG_FORCE_TENSOR
    _clear(layer)
    for _ in range(3):                             # several launches: every SM gets a CTA again
        y = layer(xs)
    torch.cuda.synchronize()
    assert torch.equal(y, want) and _status(layer) == (0, 0)
    _, yex = O.reference_forward(x, q, s, z, 4)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()
