"""Compatibility package: ``import custom_models`` registers ``ipttcdv9`` and ``ipttt`` with the HF
Auto* factories, exactly as the reference package of the same name does (custom_models/__init__.py)."""
from ttcd_b200 import models as _models

from . import ipttcd, ipttt  # noqa: F401

_models.register_all()
