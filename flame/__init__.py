"""Compatibility package: ``python -m flame.train`` and ``python -m flame.utils.convert_*`` are the public
entry points of the reference repository; here they dispatch to the ttcd_b200 implementation."""
__version__ = "0.1.0"
