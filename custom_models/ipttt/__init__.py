from ttcd_b200.models import IPTTTConfig, IPTTTForCausalLM, IPTTTModel  # noqa: F401

__all__ = ["IPTTTConfig", "IPTTTModel", "IPTTTForCausalLM"]
