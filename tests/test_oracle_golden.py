"""The oracle against fixtures generated from the reference's own Python
(tests/golden/make_golden.py): packed layout, zero-point handling, dequant,
fp16 matmul and the fp16->codes front end."""
import os

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_reference_layout_matches_fixture(golden_dir, bits):
    f = _load(golden_dir, f"pack_b{bits}.npz")
    K, N, GS = int(f["K"]), int(f["N"]), int(f["GS"])
    args = {"K": K, "N": N, "NBITS": bits, "GS": GS}
    w, s, z = O.ref_convert_params(args, (f["q"], f["s"], f["z"]))
    assert w.dtype == np.int8 and w.shape == (N, K * bits // 8)
    np.testing.assert_array_equal(w, f["w_asym"])
    np.testing.assert_array_equal(s.view(np.uint16), f["s_asym"].view(np.uint16))
    np.testing.assert_array_equal(z, f["z_asym"])
    w2, s2, z2 = O.ref_convert_params(args, (f["q"], f["s"], None))
    assert z2 is None
    np.testing.assert_array_equal(w2, f["w_sym"])
    w3 = O.ref_convert_params({"K": K, "N": N, "NBITS": bits}, (f["q"],))
    np.testing.assert_array_equal(w3, f["w_groupless"])


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_reference_layout_round_trip(golden_dir, bits):
    f = _load(golden_dir, f"pack_b{bits}.npz")
    np.testing.assert_array_equal(O.ref_unpack_weight(f["w_asym"], bits), f["q"])
    # zeros come back as the effective (z+1, clamped) values the kernel subtracts
    ze = O.ref_unpack_zero(f["z_asym"], bits)
    np.testing.assert_array_equal(ze, np.minimum(f["z"] + 1, (1 << bits) - 1))
    assert ze[0, 0] == (1 << bits) - 1 and ze[0, 1] == 1


def test_convert_arity_errors():
    q = np.zeros((64, 8), dtype=np.int32)
    with pytest.raises(ValueError):
        O.ref_convert_params({"K": 64, "N": 8, "NBITS": 4, "GS": 32}, (q,))
    with pytest.raises(ValueError):
        O.ref_convert_params({"K": 64, "N": 8, "NBITS": 4}, (q, q))
    with pytest.raises(KeyError):
        O.ref_permute_order(3)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_dequant_and_matmul_match_fixture(golden_dir, bits):
    f = _load(golden_dir, f"dequant_b{bits}.npz")
    wd = O.dequant_unclamped(f["q"], f["s"], f["z"])
    np.testing.assert_array_equal(wd.numpy().view(np.uint16), f["wdq"].view(np.uint16))
    # effective-zero form agrees wherever the clamp is not in play (z < 2^b-1 here)
    we = O.dequant_effective(f["q"], f["s"], O.effective_zero(f["z"], bits))
    np.testing.assert_array_equal(we.numpy().view(np.uint16), f["wdq"].view(np.uint16))
    y = O.qlinear_fp16(f["x"], wd)
    np.testing.assert_array_equal(y.numpy().view(np.uint16), f["y"].view(np.uint16))
    yg = O.gemv_groupless_fp16(f["x"], f["q"])
    np.testing.assert_array_equal(yg.numpy().view(np.uint16), f["y_groupless"].view(np.uint16))
    # the float64 contraction is what both approximate
    ye = O.qlinear_exact(f["x"], wd)
    assert np.abs(ye - f["y"].astype(np.float64)).max() <= 1e-2 * np.abs(ye).max()


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_clamp_differs_only_at_top_zero(bits):
    x, q, s, z = O.make_case(1, 16, 256, bits, 64, seed=5)
    z.clamp_(max=(1 << bits) - 2)
    z[0, :] = (1 << bits) - 1
    a = O.dequant_unclamped(q, s, z).float()
    b = O.dequant_effective(q, s, O.effective_zero(z.numpy(), bits)).float()
    diff = (a - b).abs()
    assert torch.all(diff[64:] == 0)
    # one scale step (up to fp16 rounding of the two products) in the clamped group
    assert torch.allclose(diff[:64], s[0].float().expand(64, -1), rtol=0, atol=6e-3)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_asymmetric_quant_matches_fixture(golden_dir, bits):
    f = _load(golden_dir, f"quant_b{bits}.npz")
    q, s, z = O.asymmetric_quant(torch.from_numpy(f["w"]), int(f["GS"]), bits)
    np.testing.assert_array_equal(q.numpy(), f["q"])
    np.testing.assert_array_equal(s.numpy().view(np.uint16), f["s"].view(np.uint16))
    np.testing.assert_array_equal(z.numpy(), f["z"])
    wd = O.dequant_unclamped(q, s, z)
    np.testing.assert_array_equal(wd.numpy().view(np.uint16), f["wdq"].view(np.uint16))


def test_algorithmic_bytes_config0():
    # 2(MK+MN) + NK/2 + 32*4096*2 + 32*4096/2 for M=1, N=K=4096, W4 g128 asym
    assert O.algorithmic_bytes(1, 4096, 4096, 4, 128, False) == 8_732_672
    assert O.algorithmic_bytes(1, 4096, 4096, 4, -1, True) == 16384 + 8_388_608
