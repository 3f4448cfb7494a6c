"""``python -m flame.train --job.config_file ... --model.config ...`` (same flags as the reference trainer)."""
from ttcd_b200.train.config_manager import JobConfig
from ttcd_b200.train.trainer import cli, main  # noqa: F401

if __name__ == "__main__":
    cli()
