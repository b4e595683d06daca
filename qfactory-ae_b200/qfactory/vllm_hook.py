"""vLLM linear-method hook: `--quantization qfactory`.

Same classes and methods as the reference's patch against vLLM
(reference: third_party/vllm-qfactory.patch:66-214): `QFactoryConfig` reads `bits` and
`group_size` from the checkpoint's quantization config, `QFactoryLinearMethod.create_weights`
registers the GPTQ-format parameters, `process_weights_after_loading` builds `layer.qlinear`,
`apply` calls it and adds the bias.  Two differences: the loaded GPTQ tensors are really
repacked into the B200 layout (the reference allocated uninitialised buffers and skipped
weight loading, patch :188-203, :223-228), and the layer serves any batch size.

The tensor-parallel all-reduce stays where vLLM has it (RowParallelLinear.forward); the hook
itself never communicates.  vLLM is imported lazily: `register()` needs it, the repacking
helpers do not.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .gptq import check_g_idx, layer_from_gptq

QUANT_NAME = "qfactory"


def build_classes():
    """Create the config / method classes against the installed vLLM and return them."""
    from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase
    from vllm.model_executor.layers.quantization.base_config import QuantizationConfig
    from vllm.model_executor.parameter import GroupQuantScaleParameter, PackedvLLMParameter, RowvLLMParameter

    class QFactoryConfig(QuantizationConfig):
        """Config class for QFactory (reference: patch :66-111)."""

        def __init__(self, weight_bits: int, group_size: int, sym: bool = False):
            super().__init__()
            self.weight_bits = weight_bits
            self.pack_factor = 32 // weight_bits
            self.group_size = group_size
            self.sym = sym

        @classmethod
        def from_config(cls, config: Dict[str, Any]) -> "QFactoryConfig":
            return cls(cls.get_from_keys(config, ["bits"]), cls.get_from_keys(config, ["group_size"]),
                       bool(cls.get_from_keys_or(config, ["sym"], False)))

        @classmethod
        def override_quantization_method(cls, hf_quant_cfg, user_quant) -> Optional[str]:
            return user_quant if user_quant == QUANT_NAME else None

        @classmethod
        def get_min_capability(cls) -> int:
            return 100  # sm_100a kernels only

        @classmethod
        def get_supported_act_dtypes(cls) -> List[torch.dtype]:
            return [torch.float16]

        def get_quant_method(self, layer: torch.nn.Module, prefix: str):
            return QFactoryLinearMethod(self, prefix) if isinstance(layer, LinearBase) else None

        @classmethod
        def get_name(cls) -> str:
            return QUANT_NAME

        @staticmethod
        def get_config_filenames() -> List[str]:
            raise NotImplementedError

    class QFactoryLinearMethod(LinearMethodBase):
        """Linear method for QFactory (reference: patch :113-214)."""

        def __init__(self, quant_config, prefix: str = ""):
            self.quant_config = quant_config
            self.prefix = prefix

        def create_weights(self, layer, input_size_per_partition: int, output_partition_sizes: List[int],
                           input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs):
            cfg = self.quant_config
            n = sum(output_partition_sizes)
            loader = extra_weight_attrs.get("weight_loader")
            groups = input_size_per_partition // cfg.group_size
            layer.register_parameter("qweight", PackedvLLMParameter(
                data=torch.empty(input_size_per_partition // cfg.pack_factor, n, dtype=torch.int32),
                input_dim=0, output_dim=1, packed_dim=0, packed_factor=cfg.pack_factor, weight_loader=loader))
            layer.register_parameter("g_idx", RowvLLMParameter(
                data=torch.empty(input_size_per_partition, dtype=torch.int32), input_dim=0, weight_loader=loader))
            layer.register_parameter("scales", GroupQuantScaleParameter(
                data=torch.empty(groups, n, dtype=params_dtype), input_dim=0, output_dim=1, weight_loader=loader))
            layer.register_parameter("qzeros", PackedvLLMParameter(
                data=torch.empty(groups, n // cfg.pack_factor, dtype=torch.int32),
                input_dim=0, output_dim=1, packed_dim=1, packed_factor=cfg.pack_factor, weight_loader=loader))

        def process_weights_after_loading(self, layer) -> None:
            layer.qlinear = repack_loaded_layer(layer, self.quant_config.weight_bits, self.quant_config.group_size,
                                                self.quant_config.sym)
            for name in ("qweight", "qzeros", "scales", "g_idx"):
                layer.register_parameter(name, None)

        def apply(self, layer, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
            out = layer.qlinear(x)
            if bias is not None:
                out.add_(bias)
            return out

    return QFactoryConfig, QFactoryLinearMethod


def repack_loaded_layer(layer, bits: int, group_size: int, sym: bool = False):
    """GPTQ parameters of a loaded vLLM layer -> packed QLinear (K, N per tensor-parallel
    partition come from the parameter shapes, as in the reference hook, patch :188-200)."""
    g_idx = getattr(layer, "g_idx", None)
    if g_idx is not None:
        g = g_idx.data
        # row-parallel shards carry global group indices: only the pattern inside the shard matters
        g = g - g.min()
        if not check_g_idx(g, group_size):
            raise ValueError("activation-reordered GPTQ checkpoints (desc_act=True) are not supported")
    return layer_from_gptq(layer.qweight.data, layer.qzeros.data, layer.scales.data, bits, group_size, None, sym)


def register():
    """Register the method with vLLM's quantization registry under the name `qfactory`."""
    from vllm.model_executor.layers.quantization import register_quantization_config

    QFactoryConfig, _ = build_classes()
    return register_quantization_config(QUANT_NAME)(QFactoryConfig)
