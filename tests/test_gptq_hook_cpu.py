"""CPU tests of the GPTQ checkpoint ingestion used by the vLLM hook."""
import types

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import gptq, layout, vllm_hook


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_gptq_word_packing_round_trip(bits):
    g = torch.Generator().manual_seed(bits)
    K, N, GS = 256, 64, 128
    q = torch.randint(0, 1 << bits, (K, N), generator=g, dtype=torch.int32)
    z = torch.randint(0, 1 << bits, (K // GS, N), generator=g, dtype=torch.int32)
    qw, qz = gptq.pack_qweight(q, bits), gptq.pack_qzeros(z, bits)
    assert qw.shape == (K * bits // 32, N) and qz.shape == (K // GS, N * bits // 32)
    assert torch.equal(gptq.unpack_qweight(qw, bits), q)
    assert torch.equal(gptq.unpack_qzeros(qz, bits), z)
    # code k of a word sits at bits [(k % pf) * bits, +bits): check one word by hand
    pf = 32 // bits
    word = sum(int(q[j, 0]) << (j * bits) for j in range(pf)) & 0xFFFFFFFF
    assert (int(qw[0, 0]) & 0xFFFFFFFF) == word


def test_layer_from_gptq_holds_the_same_codes_scales_and_effective_zeros():
    bits, K, N, GS = 4, 512, 128, 128
    x, q, s, z = O.make_case(1, N, K, bits, GS, False, seed=4)
    layer = gptq.layer_from_gptq(gptq.pack_qweight(q, bits), gptq.pack_qzeros(z, bits), s, bits, GS,
                                 g_idx=torch.arange(K, dtype=torch.int32) // GS)
    q2, s2, z2 = layer.unpack_torch()  # whatever layout the factory picked
    assert torch.equal(q2, q)
    assert np.array_equal(z2.numpy(), O.effective_zero(z.numpy(), bits))
    assert torch.equal(s2.view(torch.int16), s.view(torch.int16))


def test_activation_reordered_checkpoints_are_rejected():
    bits, K, N, GS = 4, 256, 128, 128
    x, q, s, z = O.make_case(1, N, K, bits, GS, False, seed=5)
    g_idx = torch.randperm(K, dtype=torch.int32) // GS
    with pytest.raises(ValueError):
        gptq.layer_from_gptq(gptq.pack_qweight(q, bits), gptq.pack_qzeros(z, bits), s, bits, GS, g_idx=g_idx)


def test_repack_of_a_loaded_row_parallel_shard():
    # a row-parallel shard carries GLOBAL group ids in g_idx: only the pattern inside the shard counts
    bits, K, N, GS = 4, 256, 128, 128
    x, q, s, z = O.make_case(1, N, K, bits, GS, False, seed=6)
    P = lambda t: types.SimpleNamespace(data=t)
    fake = types.SimpleNamespace(qweight=P(gptq.pack_qweight(q, bits)), qzeros=P(gptq.pack_qzeros(z, bits)),
                                 scales=P(s), g_idx=P(torch.arange(K, dtype=torch.int32) // GS + 6))
    layer = vllm_hook.repack_loaded_layer(fake, bits, GS)
    assert layer.in_features == K and layer.out_features == N
    assert torch.equal(layer.unpack_torch()[0], q)


def test_hook_classes_build_against_the_installed_vllm():
    pytest.importorskip("vllm")
    try:
        Config, Method = vllm_hook.build_classes()
    except Exception as e:  # vLLM present but not importable without a GPU runtime
        pytest.skip(f"vLLM internals not importable here: {e}")
    cfg = Config.from_config({"bits": 4, "group_size": 128})
    assert cfg.get_name() == "qfactory" and cfg.pack_factor == 8 and cfg.group_size == 128
    assert Config.override_quantization_method({}, "qfactory") == "qfactory"
    assert Config.override_quantization_method({}, "gptq") is None
    assert torch.float16 in cfg.get_supported_act_dtypes()
    for name in ("create_weights", "process_weights_after_loading", "apply"):
        assert hasattr(Method, name)
