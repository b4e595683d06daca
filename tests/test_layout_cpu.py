"""CPU tests of the host-side logic: the packed layout, the packing entry point's
contract, the fp16 front end, and that the C-ABI library loads and exports every symbol
the public header declares.  No kernel is launched here."""
import os
import re

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from oracle import qf_oracle as O
from qfactory import _native, layout
from qfactory.convert import convert_params, unpack_params
from qfactory.quantize import asymmetric_quant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("N", [1, 127, 128, 200, 384])
def test_pack_round_trip_exact(bits, N):
    K = 512
    g = torch.Generator().manual_seed(bits * 1000 + N)
    q = torch.randint(0, 1 << bits, (K, N), generator=g, dtype=torch.int32)
    w = layout.pack_weight(q, bits)
    assert w.dtype == torch.int8 and w.shape == (layout.padded_rows(N), K * bits // 8)
    assert torch.equal(layout.unpack_weight(w, N, K, bits), q)


@settings(max_examples=25, deadline=None)
@given(bits=st.sampled_from([2, 3, 4, 8]), n=st.integers(1, 300), ku=st.integers(1, 6), seed=st.integers(0, 2**31 - 1))
def test_pack_round_trip_property(bits, n, ku, seed):
    K = 128 * ku
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 1 << bits, (K, n), generator=g, dtype=torch.int32)
    assert torch.equal(layout.unpack_weight(layout.pack_weight(q, bits), n, K, bits), q)


@settings(max_examples=20, deadline=None)
@given(bits=st.sampled_from([2, 3, 4, 8]), n=st.integers(1, 300), ku=st.integers(1, 4), seed=st.integers(0, 2**31 - 1))
def test_fragment_pack_round_trip_property(bits, n, ku, seed):
    """The fragment layout of every bit width (3-bit: placed bit by bit, one field pair in the spare
    bits) holds the same codes: pack -> unpack is the identity, the padded rows are zero, and every
    byte of the packed tensor is used (packing all-ones codes sets every bit of the real rows)."""
    K = 128 * ku
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 1 << bits, (K, n), generator=g, dtype=torch.int32)
    w = layout.pack_weight_fragment(q, bits)
    assert w.dtype == torch.int8 and w.shape == (layout.padded_rows(n), K * bits // 8)
    assert torch.equal(layout.unpack_weight_fragment(w, n, K, bits), q)
    ones = layout.pack_weight_fragment(torch.full((K, n), (1 << bits) - 1, dtype=torch.int32), bits)
    set_bits = int(layout._bytes_to_words(ones.view(torch.uint8).reshape(-1, 4)).to(torch.int64).apply_(lambda v: bin(v & 0xFFFFFFFF).count("1")).sum())
    assert set_bits == K * n * bits


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_word_field_order_is_the_reference_permutation(bits):
    # one row, one 32-bit word: the word must equal the reference packer's word for the same codes
    assert layout.field_elements(bits) == O.ref_permute_order(bits)
    pf = 32 // bits
    K = layout.unit_k(bits) * 4  # >= 64
    q = torch.arange(K, dtype=torch.int32).remainder(1 << bits).reshape(K, 1)
    mine = layout.pack_weight(q, bits).view(torch.uint8)[0]  # tile 0, vectors along K, row 0 -> first 16 bytes
    first_vec = layout.pack_weight(q, bits).view(torch.uint8).view(1, K // layout.unit_k(bits), 128, 16)[0, 0, 0]
    ref = O.ref_pack_weight(q.numpy(), bits).view(np.uint8)[0]
    assert np.array_equal(first_vec.numpy(), ref[:16])
    assert mine.numel() == K * bits // 8


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_new_layout_holds_the_same_codes_as_the_reference_layout(golden_dir, bits):
    f = np.load(os.path.join(golden_dir, f"pack_b{bits}.npz"))
    K, N, GS = int(f["K"]), int(f["N"]), int(f["GS"])
    args = {"K": K, "N": N, "NBITS": bits, "GS": GS}
    w, s, z = convert_params(args, (torch.from_numpy(f["q"]), torch.from_numpy(f["s"]), torch.from_numpy(f["z"])))
    q2, s2, z2 = unpack_params(args, (w, s, z))
    assert np.array_equal(q2.numpy(), O.ref_unpack_weight(f["w_asym"], bits))
    assert np.array_equal(z2.numpy(), O.ref_unpack_zero(f["z_asym"], bits))  # effective zeros, clamp included
    assert np.array_equal(s2.numpy().view(np.uint16), f["s_asym"].T.view(np.uint16))
    # symmetric and group-less forms
    w3, s3, z3 = convert_params(args, (torch.from_numpy(f["q"]), torch.from_numpy(f["s"]), None))
    assert z3 is None and torch.equal(w3, w)
    w4 = convert_params({"K": K, "N": N, "NBITS": bits}, (torch.from_numpy(f["q"]),))
    assert torch.equal(w4, w)


def test_convert_params_contract():
    q = torch.zeros(128, 8, dtype=torch.int32)
    s = torch.ones(2, 8, dtype=torch.float16)
    z = torch.zeros(2, 8, dtype=torch.int32)
    with pytest.raises(ValueError):
        convert_params({"K": 128, "N": 8, "NBITS": 4, "GS": 64}, (q,))
    with pytest.raises(ValueError):
        convert_params({"K": 128, "N": 8, "NBITS": 4}, (q, s, z))
    with pytest.raises(AssertionError):
        convert_params({"K": 128, "N": 8, "NBITS": 4, "GS": 64}, (q + 16, s, z))  # code out of range
    with pytest.raises(AssertionError):
        convert_params({"K": 128, "N": 8, "NBITS": 4, "GS": 64}, (q, s.float(), z))  # scale dtype
    with pytest.raises(AssertionError):
        convert_params({"K": 128, "N": 8, "NBITS": 4, "GS": 64}, (q.long(), s, z))  # weight dtype
    with pytest.raises(AssertionError):
        convert_params({"K": 128, "N": 8, "NBITS": 4, "GS": 64}, (q, s, z - 1))  # zero out of range
    with pytest.raises(AssertionError):
        convert_params({"K": 128, "N": 9, "NBITS": 4, "GS": 64}, (q, s, z))  # shape
    with pytest.raises(ValueError):
        convert_params({"K": 128, "N": 8, "NBITS": 5, "GS": 64}, (q, s, z))
    w, s2, z2 = convert_params({"K": 128, "N": 8, "NBITS": 4, "GS": 64}, (q, s, z))
    assert w.shape == (128, 64) and s2.shape == (128, 2) and z2.shape == (128, 2)
    assert int(z2.view(torch.uint8)[0, 0]) == 1  # stored zero is z + 1
    assert int(z2.view(torch.uint8)[8, 0]) == 0  # padded rows are zero


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_zero_clamp_matches_reference_packer(bits):
    z = torch.arange(1 << bits, dtype=torch.int32).reshape(1, -1).repeat(2, 1)
    ze = layout.effective_zero(z, bits)
    assert np.array_equal(ze.numpy(), O.effective_zero(z.numpy(), bits))
    assert int(ze.max()) == (1 << bits) - 1 and int(ze.min()) == 1


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_asymmetric_quant_matches_fixture(golden_dir, bits):
    f = np.load(os.path.join(golden_dir, f"quant_b{bits}.npz"))
    q, s, z = asymmetric_quant(torch.from_numpy(f["w"]), int(f["GS"]), bits)
    assert np.array_equal(q.numpy(), f["q"])
    assert np.array_equal(s.numpy().view(np.uint16), f["s"].view(np.uint16))
    assert np.array_equal(z.numpy(), f["z"])


def test_library_loads_and_exports_every_declared_symbol():
    L = _native.lib()
    assert L.qfb_version() >= 100
    header = open(os.path.join(ROOT, "include", "qfactory_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(qfb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in the header but not exported"
    for name in _native.EXPORTS:
        assert name in declared, f"{name} bound in Python but not declared in the header"


def test_size_queries_and_status_strings():
    L = _native.lib()
    assert L.qfb_packed_weight_bytes(4096, 4096, 4) == 4096 * 4096 // 2
    assert L.qfb_packed_weight_bytes(100, 256, 3) == 128 * 256 * 3 // 8
    assert L.qfb_packed_weight_bytes(4096, 4000, 4) == 0  # K not a multiple of 64
    assert L.qfb_packed_scale_bytes(4096, 4096, 128) == 4096 * 32 * 2
    assert L.qfb_packed_zero_bytes(4096, 4096, 128) == 4096 * 32
    assert L.qfb_workspace_bytes(1, 4096, 4096, 4) > 0
    assert L.qfb_status_string(0) == b"ok" and L.qfb_status_string(2) == b"bad shape"
    assert L.qfb_select_kernel(1, 4096, 4096, 4, 0) == 1
    assert L.qfb_select_kernel(1, 4096, 4096, 5, 0) == 0


def test_argument_validation_without_a_gpu():
    # validation happens before any CUDA call, so these statuses are observable on a CPU-only host
    import ctypes

    L = _native.lib()
    d = _native.QfbLayer(None, None, None, 128, 128, 4, 64)
    assert L.qfb_linear_forward(ctypes.byref(d), None, 1, None, None, 0, 0, None) == 1  # null pointer
    d = _native.QfbLayer(16, 16, None, 128, 100, 4, 64)
    assert L.qfb_linear_forward(ctypes.byref(d), 16, 1, 16, None, 0, 0, None) == 2  # bad shape
    d = _native.QfbLayer(16, 16, None, 128, 128, 5, 64)
    assert L.qfb_linear_forward(ctypes.byref(d), 16, 1, 16, None, 0, 0, None) == 3  # unsupported bits
    d = _native.QfbLayer(24, 16, None, 128, 128, 4, 64)
    assert L.qfb_linear_forward(ctypes.byref(d), 16, 1, 16, None, 0, 0, None) == 4  # misaligned
    d = _native.QfbLayer(16, 16, None, 128, 128, 4, 64)
    assert L.qfb_linear_forward(ctypes.byref(d), 16, 0, 16, None, 0, 0, None) == 0  # empty batch is a no-op


def test_module_refuses_to_run_without_cuda():
    from qfactory import QLinear

    q = torch.zeros(128, 8, dtype=torch.int32)
    layer = QLinear.init(1, 128, 8, 4, q, 64, torch.ones(2, 8, dtype=torch.float16), torch.zeros(2, 8, dtype=torch.int32))
    assert set(layer.state_dict()) == {"w", "s", "z", "_extra_state"}  # packed tensors + the layout tag
    if not torch.cuda.is_available():
        with pytest.raises(_native.NativeError):
            layer(torch.zeros(1, 128, dtype=torch.float16))
    with pytest.raises(NotImplementedError):
        QLinear.init(1, 128, 8, 4, q, 64, torch.ones(2, 8, dtype=torch.float16), None, bias=True)
