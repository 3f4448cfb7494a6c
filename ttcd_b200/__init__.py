"""ttcd_b200: Blackwell-native IP-TTCD training and prefill framework."""
__version__ = "0.1.0"

from . import models, ops  # noqa: F401  (importing models registers the HF Auto* classes)
