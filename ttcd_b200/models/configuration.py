"""HF configuration classes for the three model families.

The field names, defaults and validation rules are the public surface shared
with the reference (custom_models/ipttcd/configuration_ipttcd.py:9-166,
configuration_ipttcdv8.py:10-45, configuration_ipttcdv9.py:10-35,
custom_models/ipttt/configuration_ipttt.py, and
fla/models/transformer/configuration_transformer.py), so a config JSON written
for the reference loads here unchanged.  The implementation is table driven:
each family lists ``(name, default)`` pairs, a shared initialiser assigns them,
and per-family ``_validate`` hooks run afterwards.
"""
from __future__ import annotations

import warnings
from typing import Any

from transformers.configuration_utils import PretrainedConfig

# Fields common to every decoder family (sliding-window transformer backbone).
_BACKBONE_FIELDS: tuple[tuple[str, Any], ...] = (
    ("hidden_size", 2048),
    ("num_hidden_layers", 24),
    ("num_heads", 32),
    ("num_kv_heads", None),
    ("head_dim", None),
    ("qkv_bias", False),
    ("qk_norm", False),
    ("window_size", None),
    ("rope_theta", 10000.0),
    ("rope_scaling", None),
    ("max_position_embeddings", 2048),
    ("hidden_ratio", 4),
    ("intermediate_size", None),
    ("hidden_act", "swish"),
    ("initializer_range", 0.02),
    ("elementwise_affine", True),
    ("norm_eps", 1e-6),
    ("use_cache", True),
    ("fuse_norm", True),
    ("fuse_swiglu", True),
    ("fuse_cross_entropy", True),
    ("fuse_linear_cross_entropy", False),
    ("use_l2warp", False),
    ("vocab_size", 32000),
    ("use_output_gate", False),
    ("gate_fn", "sigmoid"),
    ("gate_logit_normalizer", 16),
    ("use_flash_attn_3", False),
    ("use_l2_softmax", False),
)

_SPECIAL_TOKEN_FIELDS = (
    ("pad_token_id", None),
    ("bos_token_id", 1),
    ("eos_token_id", 2),
    ("tie_word_embeddings", False),
)


def resolve_intermediate_size(hidden_size: int, hidden_ratio: int | None, intermediate_size: int | None) -> int:
    """SwiGLU width: explicit value, else 2/3 * ratio * hidden rounded up to 256."""
    if intermediate_size is not None:
        return int(intermediate_size)
    ratio = 4 if hidden_ratio is None else hidden_ratio
    width = int(hidden_size * ratio * 2 / 3)
    return 256 * ((width + 255) // 256)


class _TableConfig(PretrainedConfig):
    """PretrainedConfig whose fields come from ``FIELDS`` tables along the MRO."""

    FIELDS: tuple[tuple[str, Any], ...] = ()
    keys_to_ignore_at_inference = ["past_key_values"]

    @classmethod
    def _field_table(cls) -> dict[str, Any]:
        table: dict[str, Any] = {}
        for klass in reversed(cls.__mro__):
            for name, default in klass.__dict__.get("FIELDS", ()):
                table[name] = default
        return table

    def __init__(self, **kwargs):
        table = self._field_table()
        for name, default in table.items():
            value = kwargs.pop(name, default)
            if isinstance(default, list) and value is not None:
                value = list(value)
            setattr(self, name, value)
        special = {name: kwargs.pop(name, default) for name, default in _SPECIAL_TOKEN_FIELDS}
        self._normalise()
        self._validate()
        super().__init__(**special, **kwargs)
        # transformers >= 5 may not keep these as attributes when passed to super
        for name, value in special.items():
            if not hasattr(self, name):
                setattr(self, name, value)

    # hooks -----------------------------------------------------------------
    def _normalise(self) -> None:
        pass

    def _validate(self) -> None:
        if self.fuse_cross_entropy and self.fuse_linear_cross_entropy:
            raise ValueError(
                "`fuse_cross_entropy` and `fuse_linear_cross_entropy` cannot be True at the same time."
            )
        if self.fuse_linear_cross_entropy:
            warnings.warn(
                "`fuse_linear_cross_entropy` is enabled: logits are never materialised and the "
                "loss is computed from bf16 logits tiles; disable it if the loss diverges.",
                stacklevel=3,
            )

    # derived ---------------------------------------------------------------
    @property
    def resolved_head_dim(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_size // self.num_heads

    @property
    def resolved_kv_heads(self) -> int:
        return self.num_heads if self.num_kv_heads is None else self.num_kv_heads

    @property
    def resolved_intermediate_size(self) -> int:
        return resolve_intermediate_size(self.hidden_size, self.hidden_ratio, self.intermediate_size)


class TransformerConfig(_TableConfig):
    """Plain (optionally sliding-window) transformer baseline, model_type ``transformer``."""

    model_type = "transformer"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)
    FIELDS = _BACKBONE_FIELDS


def _check_ttt_common(cfg) -> None:
    if any(layer < 0 or layer >= cfg.num_hidden_layers for layer in cfg.ttt_layers):
        raise ValueError("`ttt_layers` must be within `[0, num_hidden_layers)`.")
    if cfg.ttt_chunk <= 0:
        raise ValueError("`ttt_chunk` must be > 0.")
    if cfg.ttt_lr < 0:
        raise ValueError("`ttt_lr` must be >= 0.")


class IPTTTConfig(_TableConfig):
    """IP-TTT: single attention, fast weights driven by hidden states or embeddings."""

    model_type = "ipttt"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)
    FIELDS = _BACKBONE_FIELDS + (
        ("ttt_mode", False),
        ("ttt_layers", []),
        ("ttt_chunk", 8192),
        ("ttt_lr", 0.3),
        ("ttt_proj", True),
        ("ttt_proj_init", "diagonal_gaussian"),
        ("ttt_target", "hidden"),
        ("ttt_conv", True),
        ("ttt_conv_causal", False),
        ("ttt_conv_kernel_size", 5),
        ("ttt_activation_conv", False),
    )
    _TARGET_ALIASES = {
        "input_embed": "embedding",
        "input_embeds": "embedding",
        "embed": "embedding",
        "hidden_states": "hidden",
        "hidden_state": "hidden",
    }

    def _normalise(self) -> None:
        self.ttt_layers = list(self.ttt_layers) if self.ttt_layers is not None else []
        self.ttt_proj_init = str(self.ttt_proj_init)
        target = str(self.ttt_target)
        self.ttt_target = self._TARGET_ALIASES.get(target, target)
        self.ttt_conv_kernel_size = int(self.ttt_conv_kernel_size)
        self.ttt_activation_conv = bool(self.ttt_activation_conv)

    def _validate(self) -> None:
        _check_ttt_common(self)
        if self.ttt_proj_init not in {"diagonal", "diagonal_gaussian", "zero"}:
            raise ValueError("`ttt_proj_init` must be one of {'diagonal', 'diagonal_gaussian', 'zero'}.")
        # "layer_input" (the residual stream entering the block) is what the HF-Llama inference port of the reference
        # feeds its fast weights (custom_models/ipttt/inference.py:783-816); the training model knows the other two
        if self.ttt_target not in {"hidden", "embedding", "layer_input"}:
            raise ValueError("`ttt_target` must be one of {'hidden', 'embedding'}.")
        if self.ttt_conv_kernel_size <= 0 or self.ttt_conv_kernel_size % 2 == 0:
            raise ValueError("`ttt_conv_kernel_size` must be a positive odd integer.")
        super()._validate()


class IPTTCDConfig(_TableConfig):
    """Base IP-TTCD fields (teacher/student dual attention + fast-weight distillation)."""

    model_type = "ipttcd"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)
    FIELDS = _BACKBONE_FIELDS + (
        ("ttt_mode", False),
        ("ttt_layers", []),
        ("ttt_chunk", 8192),
        ("ttt_lr", 0.3),
        ("ttt_proj", True),
        ("ttt_proj_init", "diagonal"),
        ("ttt_conv", False),
        ("ttt_proj_diff_use_wcur", True),
        ("ttt_detach_wcur_in_proj_diff", False),
        ("dynamic_lr", True),
        ("ttt_visible_chunks", 1),
        ("use_muon", False),
        ("ttt_weight_renorm", None),
        ("ttt_norm_proj", True),
        ("ttt_norm_proj_diff", False),
        ("ttt_normalize_diff_inputs", False),
        ("ttt_normalize_student_features", True),
        ("ttt_norm_log_freq", 50),
    )

    def _normalise(self) -> None:
        self.ttt_layers = list(self.ttt_layers) if self.ttt_layers is not None else []
        if self.ttt_proj_init == "zeroinit":
            self.ttt_proj_init = "zero"
        self.ttt_detach_wcur_in_proj_diff = bool(self.ttt_detach_wcur_in_proj_diff)
        # `ttt_norm_proj` is the historical name of the post-update Frobenius renorm.
        if self.ttt_weight_renorm is None:
            self.ttt_weight_renorm = bool(self.ttt_norm_proj)
        self.ttt_weight_renorm = bool(self.ttt_weight_renorm)
        self.ttt_normalize_student_features = bool(self.ttt_normalize_student_features)
        self.ttt_norm_log_freq = int(self.ttt_norm_log_freq)

    def _validate(self) -> None:
        _check_ttt_common(self)
        if self.ttt_norm_log_freq <= 0:
            raise ValueError("`ttt_norm_log_freq` must be > 0.")
        if self.ttt_proj_init not in {"diagonal", "diagonal_gaussian", "random", "zero", "ipttt"}:
            raise ValueError(
                "`ttt_proj_init` must be one of {'diagonal', 'diagonal_gaussian', 'random', 'zero', 'zeroinit', 'ipttt'}."
            )
        super()._validate()


class IPTTCDv8Config(IPTTCDConfig):
    """Adds the per-chunk depthwise teacher/student convolutions."""

    model_type = "ipttcdv8"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)
    FIELDS = (
        ("ttt_teacher_conv", True),
        ("ttt_student_conv", True),
        ("ttt_conv_kernel_size", 5),
        ("ttt_conv_causal", True),
        ("ttt_teacher_conv_init", "zero"),
        ("ttt_student_conv_init", "zero"),
        ("ttt_output_use_teacher_conv", True),
        ("ttt_output_source", "teacher"),
    )

    def _normalise(self) -> None:
        super()._normalise()
        self.ttt_teacher_conv = bool(self.ttt_teacher_conv)
        self.ttt_student_conv = bool(self.ttt_student_conv)
        self.ttt_conv_kernel_size = int(self.ttt_conv_kernel_size)
        self.ttt_conv_causal = bool(self.ttt_conv_causal)
        self.ttt_teacher_conv_init = str(self.ttt_teacher_conv_init).lower()
        self.ttt_student_conv_init = str(self.ttt_student_conv_init).lower()
        self.ttt_output_use_teacher_conv = bool(self.ttt_output_use_teacher_conv)
        self.ttt_output_source = str(self.ttt_output_source).lower()
        self.ttt_conv = bool(self.ttt_conv or self.ttt_teacher_conv or self.ttt_student_conv)

    def _validate(self) -> None:
        if self.ttt_conv_kernel_size <= 0 or self.ttt_conv_kernel_size % 2 == 0:
            raise ValueError("`ttt_conv_kernel_size` must be a positive odd integer.")
        if self.ttt_output_source not in {"teacher", "student"}:
            raise ValueError("`ttt_output_source` must be either 'teacher' or 'student'.")
        for name in ("ttt_teacher_conv_init", "ttt_student_conv_init"):
            if getattr(self, name) not in {"identity", "zero", "random"}:
                raise ValueError(f"`{name}` must be one of 'identity', 'zero', or 'random'.")
        super()._validate()


class IPTTCDv9Config(IPTTCDv8Config):
    """Off-policy update against the fixed base weight + grouped prefix scan."""

    model_type = "ipttcdv9"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)
    FIELDS = (
        ("ttt_update_every", 4),
        ("ttt_weight_renorm", False),
        ("ttt_fuse_proj_into_update", True),
        ("ttt_force_grouped_scan", False),
        ("ttt_scan_group_size", 4),
        ("ttt_scan_state_dtype", "compute"),
    )

    def _normalise(self) -> None:
        super()._normalise()
        self.ttt_update_every = int(self.ttt_update_every)
        self.ttt_fuse_proj_into_update = bool(self.ttt_fuse_proj_into_update)
        self.ttt_force_grouped_scan = bool(self.ttt_force_grouped_scan)
        self.ttt_scan_group_size = int(self.ttt_scan_group_size)
        self.ttt_scan_state_dtype = str(self.ttt_scan_state_dtype).lower()

    def _validate(self) -> None:
        if self.ttt_update_every <= 0:
            raise ValueError("`ttt_update_every` must be > 0.")
        if self.ttt_scan_group_size <= 0:
            raise ValueError("`ttt_scan_group_size` must be > 0.")
        if self.ttt_scan_state_dtype not in {"compute", "bf16", "fp32"}:
            raise ValueError("`ttt_scan_state_dtype` must be one of {'compute', 'bf16', 'fp32'}.")
        super()._validate()


class IPTTCDv9LowCopyConfig(IPTTCDv9Config):
    model_type = "ipttcdv9_lowcopy"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)


class DeltaNetBaselineConfig(IPTTCDConfig):
    """SWA transformer + training-only DeltaNet sub-layer on ``ttt_layers`` (same fields as ``ipttcd``)."""

    model_type = "deltanet_baseline"

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)


_RECURRENT_COMMON_FIELDS: tuple[tuple[str, Any], ...] = (
    ("attn_mode", "chunk"),
    ("hidden_size", 2048),
    ("use_short_conv", True),
    ("conv_size", 4),
    ("max_position_embeddings", 2048),
    ("hidden_ratio", 4),
    ("intermediate_size", None),
    ("hidden_act", "swish"),
    ("norm_eps", 1e-6),
    ("attn", None),
    ("use_cache", True),
    ("initializer_range", 0.02),
    ("fuse_norm", True),
    ("fuse_swiglu", True),
    ("fuse_cross_entropy", True),
    ("fuse_linear_cross_entropy", False),
    ("use_l2warp", False),
    ("vocab_size", 32000),
)


class _RecurrentConfig(_TableConfig):
    """Shared rules of the linear-recurrent families: the optional ``attn`` dict turns the listed layers into softmax
    attention (hybrid layouts) and must name ``layers`` and ``num_heads``."""

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)

    def _validate(self) -> None:
        super()._validate()
        attn = self.attn
        if attn is not None:
            if not isinstance(attn, dict):
                raise ValueError("attn must be a dictionary")
            if "layers" not in attn:
                raise ValueError("Layer indices must be provided to initialize hybrid attention layers")
            if "num_heads" not in attn:
                raise ValueError("Number of heads must be provided to initialize hybrid attention layers")
            attn.setdefault("num_kv_heads", attn["num_heads"])
            attn.setdefault("qkv_bias", False)
            attn.setdefault("window_size", None)
            attn.setdefault("rope_theta", 10000.0)


class DeltaNetConfig(_RecurrentConfig):
    """``delta_net`` (fla/models/delta_net/configuration_delta_net.py:8-110)."""

    model_type = "delta_net"
    FIELDS = _RECURRENT_COMMON_FIELDS + (
        ("expand_k", 1.0),
        ("expand_v", 1.0),
        ("use_gate", False),
        ("use_beta", True),
        ("use_output_norm", True),
        ("num_heads", 16),
        ("qk_norm", "l2"),
        ("qk_activation", "silu"),
        ("num_hidden_layers", 24),
    )

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)


class GatedDeltaNetConfig(_RecurrentConfig):
    """``gated_deltanet`` (fla/models/gated_deltanet/configuration_gated_deltanet.py:8-100)."""

    model_type = "gated_deltanet"
    FIELDS = _RECURRENT_COMMON_FIELDS + (
        ("expand_v", 2.0),
        ("use_gate", True),
        ("allow_neg_eigval", False),
        ("head_dim", 256),
        ("num_heads", 6),
        ("num_v_heads", None),
        ("num_hidden_layers", 21),
    )

    def __init__(self, **kwargs):  # explicit: keeps HF from generating a dataclass __init__
        super().__init__(**kwargs)


__all__ = [
    "DeltaNetBaselineConfig",
    "DeltaNetConfig",
    "GatedDeltaNetConfig",
    "TransformerConfig",
    "IPTTTConfig",
    "IPTTCDConfig",
    "IPTTCDv8Config",
    "IPTTCDv9Config",
    "IPTTCDv9LowCopyConfig",
    "resolve_intermediate_size",
]
