from ttcd_b200.models import (IPTTCDv9Config, IPTTCDv9ForCausalLM, IPTTCDv9Model)  # noqa: F401

__all__ = ["IPTTCDv9Config", "IPTTCDv9Model", "IPTTCDv9ForCausalLM"]
