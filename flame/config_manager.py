from ttcd_b200.train.config_manager import JobConfig, string_list  # noqa: F401
