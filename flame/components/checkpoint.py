from ttcd_b200.train.checkpoint import TrainState  # noqa: F401
