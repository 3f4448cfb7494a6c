from ttcd_b200.utils.convert import strip_legacy_buffers  # noqa: F401
