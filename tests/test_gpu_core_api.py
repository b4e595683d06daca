"""Operator-level API: `QMatmul(...).compile_profile()` and `Matmul(...).compile_profile()` closures
with the reference's argument order (reference: qfactory/core/matmul.py:123-146 for the grouped
closure `inner(activation, weight, output, scale, zero)` / `inner_sym(activation, weight, output,
scale)`, :240-270 for the group-less `inner(activation, weight, output)`), on tensors packed by
`convert_params`, against the oracle."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import Matmul, QMatmul, _native, layout
from qfactory.convert import convert_params

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _packed(N, K, bits, GS, sym, lay, M, seed):
    x, q, s, z = O.make_case(M, N, K, bits, GS, sym, seed)
    args = {"K": K, "N": N, "NBITS": bits, "LAYOUT": lay}
    if GS != -1:
        args["GS"] = GS
        w, ps, pz = convert_params(args, (q.cuda(), s.cuda(), None if z is None else z.cuda()))
    else:
        w, ps, pz = convert_params(args, (q.cuda(),)), None, None
    return x, q, s, z, w, ps, pz


def _check(y, x, q, s, z, bits):
    _, yex = O.reference_forward(x, q, s, z, bits)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()


@pytest.mark.parametrize("lay", ["tile", "fragment"])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [1, 16, 48])
def test_qmatmul_asymmetric_closure(lay, bits, M):
    N, K, GS = 640, 2048, 128
    x, q, s, z, w, ps, pz = _packed(N, K, bits, GS, False, lay, M, seed=bits + M)
    f = QMatmul(M, N, K, bits, False, torch.float16, torch.int8, GS, "nt", False, packed_layout=lay).compile_profile()
    out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    assert f(x.cuda(), w, out, ps, pz) == 0          # the reference closure returns the launcher's code
    want_kernel = (3 if M <= 16 else 2) if lay == "fragment" else None
    if want_kernel is not None:
        assert _native.last_launch()["kernel"] == want_kernel
    _check(out, x, q, s, z, bits)


@pytest.mark.parametrize("lay", ["tile", "fragment"])
def test_qmatmul_symmetric_closure_takes_no_zero(lay):
    M, N, K, bits, GS = 3, 384, 1024, 4, 128
    x, q, s, z, w, ps, pz = _packed(N, K, bits, GS, True, lay, M, seed=21)
    assert pz is None
    f = QMatmul(M, N, K, bits, True, torch.float16, torch.int8, group_size=GS, packed_layout=lay).compile_profile()
    out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    f(x.cuda(), w, out, ps)
    _check(out, x, q, s, None, bits)


def test_qmatmul_default_layout_follows_convert_params():
    # no layout named anywhere: the packer and the operator default to the same one
    M, N, K, bits, GS = 2, 256, 1024, 4, 128
    x, q, s, z = O.make_case(M, N, K, bits, GS, False, seed=5)
    w, ps, pz = convert_params({"K": K, "N": N, "NBITS": bits, "GS": GS}, (q.cuda(), s.cuda(), z.cuda()))
    op = QMatmul(M, N, K, bits, False, torch.float16, torch.int8, GS)
    assert op.packed_layout == layout.LAYOUT_TILE
    out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    op.compile_profile()(x.cuda(), w, out, ps, pz)
    _check(out, x, q, s, z, bits)


def test_qmatmul_validates_like_the_reference():
    M, N, K, bits, GS = 2, 256, 1024, 4, 128
    x, q, s, z, w, ps, pz = _packed(N, K, bits, GS, False, "tile", M, seed=6)
    f = QMatmul(M, N, K, bits, False, torch.float16, torch.int8, GS, packed_layout="tile").compile_profile()
    out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    with pytest.raises(AssertionError):
        f(x.cuda().float(), w, out, ps, pz)                    # activation dtype
    with pytest.raises(AssertionError):
        f(x.cuda()[:, : K // 2], w, out, ps, pz)               # activation width
    with pytest.raises(AssertionError):
        f(x.cuda(), w, out.t(), ps, pz)                        # output shape / contiguity
    with pytest.raises(AssertionError):
        QMatmul(M, N, K, bits, False, torch.float16, torch.int8, 100)   # group must divide K
    with pytest.raises(AssertionError):
        QMatmul(M, N, K, bits, False, torch.bfloat16, torch.int8, GS)


@pytest.mark.parametrize("lay", ["tile", "fragment"])
@pytest.mark.parametrize("bits", [2, 4, 8])
def test_groupless_matmul_closure_any_batch(lay, bits):
    N, K = 300, 1024
    x, q, s, z, w, _, _ = _packed(N, K, bits, -1, False, lay, 20, seed=30 + bits)
    f = Matmul(N, K, bits, packed_layout=lay).compile_profile()
    for M in (1, 7, 20):    # M is a run-time argument of the group-less closure, as in the reference
        out = torch.empty(M, N, dtype=torch.float16, device="cuda")
        f(x[:M].contiguous().cuda(), w, out)
        _check(out, x[:M], q, None, None, bits)
