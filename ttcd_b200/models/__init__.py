"""Model families and their HF Auto* registration.

Importing this package registers ``transformer``, ``ipttt``, ``ipttcdv9``, ``deltanet_baseline``, ``delta_net`` and
``gated_deltanet`` with
``AutoConfig`` / ``AutoModel`` / ``AutoModelForCausalLM`` (the reference does the same on
``import custom_models``: custom_models/ipttcd/__init__.py:17-24, custom_models/ipttt/__init__.py).
"""
from transformers import AutoConfig, AutoModel, AutoModelForCausalLM

from .configuration import (DeltaNetBaselineConfig, DeltaNetConfig, GatedDeltaNetConfig, IPTTCDConfig, IPTTCDv8Config, IPTTCDv9Config, IPTTCDv9LowCopyConfig, IPTTTConfig,
                            TransformerConfig)
from .layers import Attention, GatedMLP, RMSNorm, RotaryEmbedding, WindowKVCache
from .modeling_delta_net import (DeltaNet, DeltaNetBlock, DeltaNetForCausalLM, DeltaNetModel, GatedDeltaNet, GatedDeltaNetBlock,
                                 GatedDeltaNetForCausalLM, GatedDeltaNetModel, RecurrentCache, ShortConv)
from .modeling_deltanet_baseline import DeltaNetBaselineBlock, DeltaNetBaselineForCausalLM, DeltaNetBaselineModel
from .modeling_ipttcdv9 import IPTTCDBlock, IPTTCDForCausalLM, IPTTCDMLP, IPTTCDModel
from .modeling_ipttt import FastWeightCache, IPTTTBlock, IPTTTForCausalLM, IPTTTMLP, IPTTTModel
from .modeling_ipttt_llama import IPTTTLlamaForCausalLM, TTTDynamicCache, ipttt_config_from_llama
from .modeling_transformer import TransformerBlock, TransformerForCausalLM, TransformerModel

IPTTCDv9Model = IPTTCDModel
IPTTCDv9ForCausalLM = IPTTCDForCausalLM


def register_all() -> None:
    for cfg, model, causal in (
        (TransformerConfig, TransformerModel, TransformerForCausalLM),
        (IPTTTConfig, IPTTTModel, IPTTTForCausalLM),
        (IPTTCDv9Config, IPTTCDModel, IPTTCDForCausalLM),
        (DeltaNetBaselineConfig, DeltaNetBaselineModel, DeltaNetBaselineForCausalLM),
        (DeltaNetConfig, DeltaNetModel, DeltaNetForCausalLM),
        (GatedDeltaNetConfig, GatedDeltaNetModel, GatedDeltaNetForCausalLM),
    ):
        AutoConfig.register(cfg.model_type, cfg, exist_ok=True)
        AutoModel.register(cfg, model, exist_ok=True)
        AutoModelForCausalLM.register(cfg, causal, exist_ok=True)


register_all()

# This package's own classes by ``model_type``: the engine resolves through this table, so another package
# registering the same ``model_type`` strings with the HF Auto classes later cannot redirect it.
MODEL_CLASSES = {cfg.model_type: (cfg, causal) for cfg, causal in (
    (TransformerConfig, TransformerForCausalLM), (IPTTTConfig, IPTTTForCausalLM), (IPTTCDv9Config, IPTTCDForCausalLM),
    (DeltaNetBaselineConfig, DeltaNetBaselineForCausalLM), (DeltaNetConfig, DeltaNetForCausalLM),
    (GatedDeltaNetConfig, GatedDeltaNetForCausalLM))}

__all__ = [
    "DeltaNetConfig", "DeltaNetModel", "DeltaNetForCausalLM", "DeltaNetBlock", "DeltaNet",
    "GatedDeltaNetConfig", "GatedDeltaNetModel", "GatedDeltaNetForCausalLM", "GatedDeltaNetBlock", "GatedDeltaNet",
    "RecurrentCache", "ShortConv",
    "DeltaNetBaselineConfig", "DeltaNetBaselineModel", "DeltaNetBaselineForCausalLM", "DeltaNetBaselineBlock",
    "TransformerConfig", "IPTTTConfig", "IPTTCDConfig", "IPTTCDv8Config", "IPTTCDv9Config", "IPTTCDv9LowCopyConfig",
    "TransformerModel", "TransformerForCausalLM", "TransformerBlock",
    "IPTTTModel", "IPTTTForCausalLM", "IPTTTBlock", "IPTTTMLP", "FastWeightCache",
    "IPTTTLlamaForCausalLM", "TTTDynamicCache", "ipttt_config_from_llama",
    "IPTTCDModel", "IPTTCDForCausalLM", "IPTTCDBlock", "IPTTCDMLP", "IPTTCDv9Model", "IPTTCDv9ForCausalLM",
    "Attention", "GatedMLP", "RMSNorm", "RotaryEmbedding", "WindowKVCache", "register_all",
]
