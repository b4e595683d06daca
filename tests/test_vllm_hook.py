"""The vLLM linear-method hook executed for real: `create_weights` against the installed vLLM's
parameter classes, the registered GPTQ parameters filled through their own weight loaders,
then `process_weights_after_loading` and `apply` (reference: third_party/vllm-qfactory.patch:123-214).

The CPU part stops after the repack (the packed layer holds the checkpoint's codes, scales and
effective zeros); the GPU part runs the layer against the oracle."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from qfactory import gptq, vllm_hook

TOL = 1e-2


def _method(monkeypatch, bits=4, group_size=128):
    pytest.importorskip("vllm")
    try:
        Config, Method = vllm_hook.build_classes()
        import vllm.model_executor.parameter as vparam
    except Exception as e:
        pytest.skip(f"vLLM's linear-method classes do not import here: {e}")
    # vLLM parameters ask for the tensor-parallel rank when they are built; a bare module outside
    # an engine has no process group, so the test answers for it: rank 0 of 1
    monkeypatch.setattr(vparam, "get_tensor_model_parallel_rank", lambda: 0)
    monkeypatch.setattr(vparam, "get_tensor_model_parallel_world_size", lambda: 1)
    cfg = Config.from_config({"bits": bits, "group_size": group_size})
    return cfg, Method(cfg, "layers.0.mlp.down_proj")


def _loaded_layer(method, K, N, bits, GS, seed, device="cpu"):
    """A bare module with the hook's parameters created and filled from a seeded GPTQ 'checkpoint'."""
    x, q, s, z = O.make_case(3, N, K, bits, GS, False, seed=seed)
    layer = torch.nn.Module()
    calls = []

    def weight_loader(param, loaded, *a, **k):
        calls.append(tuple(loaded.shape))
        param.data.copy_(loaded)

    method.create_weights(layer, K, [N // 2, N // 2], K, N, torch.float16, weight_loader=weight_loader)
    pf = 32 // bits
    assert layer.qweight.shape == (K // pf, N) and layer.qweight.dtype == torch.int32
    assert layer.qzeros.shape == (K // GS, N // pf) and layer.qzeros.dtype == torch.int32
    assert layer.scales.shape == (K // GS, N) and layer.scales.dtype == torch.float16
    assert layer.g_idx.shape == (K,) and layer.g_idx.dtype == torch.int32
    ckpt = {"qweight": gptq.pack_qweight(q, bits), "qzeros": gptq.pack_qzeros(z, bits), "scales": s,
            "g_idx": (torch.arange(K) // GS).to(torch.int32)}
    for name, t in ckpt.items():
        p = getattr(layer, name)
        p.weight_loader(p, t)   # the route vLLM's loader takes
    assert len(calls) == 4
    if device != "cpu":
        layer.to(device)
    return layer, x, q, s, z


@pytest.mark.parametrize("bits", [4, 8])
def test_create_weights_and_repack_on_cpu(monkeypatch, bits):
    cfg, method = _method(monkeypatch, bits)
    K, N, GS = 512, 256, 128
    layer, x, q, s, z = _loaded_layer(method, K, N, bits, GS, seed=40 + bits)
    method.process_weights_after_loading(layer)
    assert layer.qweight is None and layer.g_idx is None  # the GPTQ tensors are released
    q2, s2, z2 = layer.qlinear.unpack_torch()
    assert torch.equal(q2, q) and torch.equal(s2.view(torch.int16), s.view(torch.int16))
    assert np.array_equal(z2.numpy(), O.effective_zero(z.numpy(), bits))


def test_activation_reordered_layer_is_rejected(monkeypatch):
    cfg, method = _method(monkeypatch)
    layer, *_ = _loaded_layer(method, 256, 128, 4, 128, seed=3)
    layer.g_idx.data.copy_(torch.randperm(256).to(torch.int32) // 128)
    with pytest.raises(ValueError):
        method.process_weights_after_loading(layer)


@pytest.mark.gpu
@pytest.mark.parametrize("with_bias", [False, True])
def test_process_weights_and_apply_against_the_oracle(monkeypatch, with_bias):
    cfg, method = _method(monkeypatch)
    K, N, GS, bits = 1024, 384, 128, 4
    layer, x, q, s, z = _loaded_layer(method, K, N, bits, GS, seed=77, device="cuda")
    method.process_weights_after_loading(layer)
    assert layer.qlinear.w.is_cuda
    x3 = torch.randn(2, 3, K, generator=torch.Generator().manual_seed(1)).half()   # 3-D activations, as vLLM passes
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2)).half() if with_bias else None
    y = method.apply(layer, x3.cuda(), None if bias is None else bias.cuda())
    assert y.shape == (2, 3, N) and y.dtype == torch.float16
    _, yex = O.reference_forward(x3.view(6, K), q, s, z, bits)
    if bias is not None:
        yex = yex + bias.double().numpy()[None, :]
    got = y.view(6, N).float().cpu().numpy().astype(np.float64)
    assert np.abs(got - yex).max() <= TOL * np.abs(yex).max()


@pytest.mark.gpu
@pytest.mark.parametrize("bits,N,K,M", [(4, 4096, 4096, 1), (4, 1024, 11008, 16), (8, 512, 2048, 5), (2, 640, 1024, 40)])
def test_layer_from_gptq_on_gpu_against_the_oracle(bits, N, K, M):
    """GPTQ checkpoint tensors (int32 words, zeros stored minus one) through the kernels."""
    GS = 128
    x, q, s, z = O.make_case(M, N, K, bits, GS, False, seed=500 + bits + M)
    layer = gptq.layer_from_gptq(gptq.pack_qweight(q, bits).cuda(), gptq.pack_qzeros(z, bits).cuda(), s.cuda(), bits, GS,
                                 g_idx=(torch.arange(K) // GS).to(torch.int32), batch_size=M)
    assert torch.equal(layer.unpack_codes().cpu(), q)   # bit-exact integer work
    y = layer(x.cuda())
    _, yex = O.reference_forward(x, q, s, z, bits)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()


@pytest.mark.gpu
def test_repack_and_forward_without_vllm():
    """The hook's repack helper on GPU tensors, with no vLLM class involved (so it still runs
    where vLLM's compiled parts fail to import)."""
    import types

    bits, K, N, GS = 4, 2048, 512, 128
    x, q, s, z = O.make_case(4, N, K, bits, GS, False, seed=9)
    P = lambda t: types.SimpleNamespace(data=t.cuda())
    fake = types.SimpleNamespace(qweight=P(gptq.pack_qweight(q, bits)), qzeros=P(gptq.pack_qzeros(z, bits)),
                                 scales=P(s), g_idx=P((torch.arange(K) // GS).to(torch.int32)))
    layer = vllm_hook.repack_loaded_layer(fake, bits, GS)
    y = layer(x.cuda())
    _, yex = O.reference_forward(x, q, s, z, bits)
    assert np.abs(y.float().cpu().numpy() - yex).max() <= TOL * np.abs(yex).max()
