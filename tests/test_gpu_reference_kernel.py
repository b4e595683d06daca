"""The reference project's OWN GPU kernel (compiled ahead of time for sm_100a from its headers by
oracle/build_ref.py, where a reference checkout was available) on the reference's own packed
layout: it pins the CPU oracle against the reference implementation itself, and this library's
kernels against both.  Skipped where the comparator library was not built."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from oracle import ref_gpu
from qfactory import QLinear

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_gpu.available(), reason="oracle/_ref/libqf_ref_gemv.so not built")]
TOL = 1e-2


@pytest.mark.parametrize("shape", [0, 1, 2, 3])
@pytest.mark.parametrize("scheduled", [0, 1])
def test_reference_kernel_oracle_and_this_library_agree(shape, scheduled):
    N, K = ref_gpu.SHAPES[shape]
    x, q, s, z = O.make_case(1, N, K, 4, 128, False, seed=shape)
    w, sp, zp = ref_gpu.pack_reference_layout(q, s, z)
    y_ref = torch.zeros(1, N, dtype=torch.float16, device="cuda")
    assert ref_gpu.launch(shape, scheduled, x.cuda(), w, y_ref, sp, zp) == 0
    torch.cuda.synchronize()
    assert ref_gpu.lib().qf_ref_last_cuda_error() == 0
    _, yex = O.reference_forward(x, q, s, z, 4)
    scale = np.abs(yex).max()
    # the reference kernel accumulates in fp16 inside a thread (qfactory/include/utils.h:179-191 of the
    # reference): it sits in the same band around the exact contraction as the fp16 CPU matmul
    assert np.abs(y_ref.float().cpu().numpy() - yex).max() <= TOL * scale
    layer = QLinear.init(1, K, N, 4, q.cuda(), 128, s.cuda(), z.cuda())
    y = layer(x.cuda())
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * scale
    assert (y.float() - y_ref.float()).abs().max().item() <= 2 * TOL * scale
