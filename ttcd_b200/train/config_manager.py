"""Job configuration: dotted command-line flags + TOML file, same names as the reference trainer.

The flag names (``--training.seq_len``, ``--checkpoint.interval`` ...), their defaults and the precedence
*command line > TOML (``--job.config_file``) > default* are the public interface of
``python -m flame.train`` in the reference (flame/config_manager.py:45-1034).  The implementation here is a
single declarative table; values are reachable as ``config.section.name``.
"""
from __future__ import annotations

import argparse
import sys
from collections import defaultdict
from types import SimpleNamespace

try:
    import tomllib
except ModuleNotFoundError:  # pragma: no cover
    import tomli as tomllib

TORCH_DTYPE_NAMES = {"float16", "float32", "bfloat16"}


def string_list(raw) -> list[str]:
    """Comma separated list; accepts an existing list (from TOML)."""
    if isinstance(raw, (list, tuple)):
        return [str(x) for x in raw]
    if raw is None or raw == "":
        return []
    return [s.strip() for s in str(raw).split(",") if s.strip()]


FLAG = "flag"          # store_true
NOFLAG = "noflag"      # store_false writing to another destination

# (dotted name, kind/type, default, help)
SPEC: list[tuple] = [
    ("job.config_file", str, None, "TOML file with job settings"),
    ("job.dump_folder", str, "./torchtitan/outputs", "folder for checkpoints, traces and logs"),
    ("job.description", str, "default job", "free-form description"),
    ("job.use_for_integration_test", FLAG, False, "accepted for compatibility; unused"),
    ("job.print_args", FLAG, False, "print the resolved configuration at start"),
    ("model.name", str, "fla", "model family registry name"),
    ("model.config", str, "fla-hub/transformer-1.3B-100B", "HF config JSON path or hub id"),
    ("model.tokenizer_path", str, "fla-hub/transformer-1.3B-100B", "tokenizer path or hub id"),
    ("model.converters", string_list, [], "model converters (float8 ...)"),
    ("model.print_after_conversion", FLAG, False, "print the model after converters ran"),
    ("profiling.enable_profiling", FLAG, False, "torch.profiler traces"),
    ("profiling.save_traces_folder", str, "profile_traces", "trace folder under dump_folder"),
    ("profiling.profile_freq", int, 10, "steps between traces"),
    ("profiling.enable_memory_snapshot", FLAG, False, "CUDA memory snapshots"),
    ("profiling.save_memory_snapshot_folder", str, "memory_snapshot", "snapshot folder under dump_folder"),
    ("optimizer.name", str, "AdamW", "AdamW or Adam"),
    ("optimizer.eps", float, 1e-8, "Adam epsilon"),
    ("optimizer.lr", float, 8e-4, "peak learning rate"),
    ("optimizer.beta1", float, 0.9, ""),
    ("optimizer.beta2", float, 0.95, ""),
    ("optimizer.weight_decay", float, 0.1, ""),
    ("optimizer.implementation", str, "fused", "for-loop | foreach | fused"),
    ("optimizer.early_step_in_backward", FLAG, False, "optimizer step inside backward hooks"),
    ("optimizer.enable_muon", FLAG, False, "Muon on 2-D hidden weights, AdamW on the rest"),
    ("optimizer.muon_momentum", float, 0.95, ""),
    ("optimizer.use_distributed_muon", FLAG, False, "all-gather variant of Muon"),
    ("lr_scheduler.warmup_steps", int, 200, ""),
    ("lr_scheduler.decay_ratio", float, None, "fraction of steps spent decaying (None = all after warmup)"),
    ("lr_scheduler.decay_type", str, "linear", "linear | sqrt | cosine"),
    ("lr_scheduler.lr_min", float, 0.0, "floor as a fraction of the peak lr"),
    ("lr_scheduler.lr_min_absolute", float, None, "floor as an absolute lr (overrides lr_min)"),
    ("lr_scheduler.anneal_begin_step", int, None, "step at which a resumed run begins its final decay"),
    ("training.batch_size", int, 8, "sequences per data-parallel rank"),
    ("training.seq_len", int, 2048, ""),
    ("training.context_len", int, 2048, "max document length with --training.varlen"),
    ("training.varlen", FLAG, False, "packed variable-length sequences (cu_seqlens)"),
    ("training.gradient_accumulation_steps", int, 1, ""),
    ("training.steps", int, 10000, ""),
    ("training.max_norm", float, 1.0, "gradient clipping norm"),
    ("training.skip_nan_inf", FLAG, False, "skip the optimizer step when the grad norm is not finite"),
    ("training.dataset", str, "HuggingFaceFW/fineweb-edu", "dataset name(s), comma separated, or mds:/path"),
    ("training.dataset_name", str, None, ""),
    ("training.dataset_split", str, None, ""),
    ("training.data_dir", str, None, ""),
    ("training.data_files", str, None, ""),
    ("training.data_probs", str, None, "sampling probabilities for several datasets"),
    ("training.streaming", FLAG, False, ""),
    ("training.shuffle_buffer_size", int, 1024, "stateful shuffle buffer; 0 disables shuffling"),
    ("training.parquet_prefetch_limit", int, 1, ""),
    ("training.parquet_range_size_mb", int, 32, ""),
    ("training.num_workers", int, 32, "dataloader workers"),
    ("training.prefetch_factor", int, 2, ""),
    ("training.pin_memory", FLAG, False, ""),
    ("training.persistent_workers", FLAG, False, ""),
    ("training.data_parallel_replicate_degree", int, 1, "HSDP replicate dimension"),
    ("training.enable_expert_parallel", FLAG, False, ""),
    ("training.data_parallel_shard_degree", int, -1, "-1 = all remaining ranks"),
    ("training.enable_cpu_offload", FLAG, False, ""),
    ("training.tensor_parallel_degree", int, 1, ""),
    ("training.disable_loss_parallel", FLAG, False, ""),
    ("training.fsdp_reshard_after_forward", str, "default",
     "default | never: bf16 weights stay resident on every rank (they fit a 180 GB GPU); always: ZeRO-3, a block's weights "
     "are stored 1/world per rank and gathered inside its first GEMM, for forward and again for backward"),
    ("training.mixed_precision_param", str, "bfloat16", ""),
    ("training.mixed_precision_reduce", str, "float32", ""),
    ("training.compile", FLAG, False, "accepted; this framework has no tracing compiler"),
    ("training.gc_freq", int, 50, "steps between Python GC runs"),
    ("training.seed", int, 42, ""),
    ("training.deterministic", FLAG, False, ""),
    ("metrics.log_freq", int, 10, ""),
    ("metrics.enable_tensorboard", FLAG, False, ""),
    ("metrics.disable_color_printing", FLAG, False, ""),
    ("metrics.save_tb_folder", str, "tb", ""),
    ("metrics.save_for_all_ranks", FLAG, False, ""),
    ("metrics.enable_wandb", FLAG, False, ""),
    ("experimental.enable_async_tensor_parallel", FLAG, False, ""),
    ("experimental.pipeline_parallel_degree", int, 1, ""),
    ("experimental.pipeline_parallel_split_points", string_list, [], ""),
    ("experimental.pipeline_parallel_schedule", str, "1F1B", ""),
    ("experimental.pipeline_parallel_schedule_csv", str, "", ""),
    ("experimental.pipeline_parallel_microbatches", int, None, ""),
    ("experimental.enable_compiled_autograd", FLAG, False, ""),
    ("experimental.context_parallel_degree", int, 1, "sequence shards (windowed K/V halo exchange)"),
    ("experimental.context_parallel_rotate_method", str, "allgather", "accepted for compatibility"),
    ("experimental.custom_model_path", str, "", "extra python package to import for model registration"),
    ("checkpoint.enable_checkpoint", FLAG, False, ""),
    ("checkpoint.folder", str, "checkpoint", ""),
    ("checkpoint.initial_load_path", str, None, "checkpoint to start from when `folder` is empty"),
    ("checkpoint.initial_load_model_weights_only", FLAG, True, ""),
    ("checkpoint.no_initial_load_model_weights_only", NOFLAG, "checkpoint.initial_load_model_weights_only", ""),
    ("checkpoint.interval", int, 500, ""),
    ("checkpoint.last_save_model_weights_only", FLAG, False, ""),
    ("checkpoint.export_dtype", str, "float32", ""),
    ("checkpoint.create_seed_checkpoint", FLAG, False, ""),
    ("checkpoint.async_mode", str, "disabled", "disabled | async | async_with_pinned_mem"),
    ("checkpoint.keep_latest_k", int, 0, ""),
    ("checkpoint.load_step", int, -1, ""),
    ("checkpoint.exclude_from_loading", string_list, [], ""),
    ("activation_checkpoint.mode", str, "selective", "none | selective | full"),
    ("activation_checkpoint.selective_ac_option", str, "2", "'op' or an integer N (every Nth block)"),
    ("activation_offload.mode", str, "none", ""),
    ("float8.enable_fsdp_float8_all_gather", FLAG, False, ""),
    ("float8.precompute_float8_dynamic_scale_for_fsdp", FLAG, False, ""),
    ("float8.force_recompute_fp8_weight_in_bwd", FLAG, False, ""),
    ("float8.recipe_name", str, None, ""),
    ("comm.init_timeout_seconds", int, 300, ""),
    ("comm.train_timeout_seconds", int, 100, ""),
    ("comm.trace_buf_size", int, 20000, ""),
    ("memory_estimation.enabled", FLAG, False, ""),
    ("memory_estimation.disable_fake_mode", FLAG, False, ""),
    ("fault_tolerance.enable", FLAG, False, ""),
    ("fault_tolerance.replica_id", int, 0, ""),
    ("fault_tolerance.group_size", int, 0, ""),
    ("fault_tolerance.min_replica_size", int, 1, ""),
]


class JobConfig:
    """Resolved configuration; ``JobConfig().parse_args(argv)`` fills sections as attributes."""

    def __init__(self):
        self.parser = argparse.ArgumentParser(description="ttcd_b200 / flame trainer arguments")
        self._defaults: dict[str, object] = {}
        self._types: dict[str, object] = {}
        for name, kind, default, helptext in SPEC:
            if kind == FLAG:
                self.parser.add_argument(f"--{name}", dest=name, action="store_true", default=default, help=helptext)
                self._defaults[name] = default
                self._types[name] = bool
            elif kind == NOFLAG:
                self.parser.add_argument(f"--{name}", dest=default, action="store_false", help=helptext)
            else:
                self.parser.add_argument(f"--{name}", dest=name, type=kind, default=default, help=helptext)
                self._defaults[name] = default
                self._types[name] = kind

    def to_dict(self) -> dict[str, dict]:
        return {k: dict(vars(v)) for k, v in vars(self).items() if isinstance(v, SimpleNamespace)}

    @staticmethod
    def _nest(flat: dict[str, object]) -> dict[str, dict]:
        out: dict[str, dict] = defaultdict(dict)
        for key, val in flat.items():
            section, name = key.split(".", 1)
            out[section][name] = val
        return out

    def parse_args(self, args_list: list[str] | None = None) -> "JobConfig":
        argv = sys.argv[1:] if args_list is None else list(args_list)
        parsed = vars(self.parser.parse_args(argv))
        merged = dict(parsed)
        toml_path = parsed.get("job.config_file")
        if toml_path:
            with open(toml_path, "rb") as fh:
                for section, values in tomllib.load(fh).items():
                    for name, val in values.items():
                        key = f"{section}.{name}"
                        typ = self._types.get(key)
                        merged[key] = string_list(val) if typ is string_list else val
            # what the user typed on the command line wins over the file
            explicit = self._explicit_args(argv)
            for key, val in explicit.items():
                merged[key] = val
        for section, values in self._nest(merged).items():
            setattr(self, section, SimpleNamespace(**values))
        self._validate()
        return self

    def _explicit_args(self, argv: list[str]) -> dict[str, object]:
        """Re-parse with every default suppressed: yields only the options present in argv."""
        aux = argparse.ArgumentParser(argument_default=argparse.SUPPRESS)
        for name, kind, default, _ in SPEC:
            if kind == FLAG:
                aux.add_argument(f"--{name}", dest=name, action="store_true")
            elif kind == NOFLAG:
                aux.add_argument(f"--{name}", dest=default, action="store_false")
            else:
                aux.add_argument(f"--{name}", dest=name, type=kind)
        ns, _ = aux.parse_known_args(argv)
        return vars(ns)

    def _validate(self) -> None:
        assert self.model.config, "--model.config is required"
        assert self.training.mixed_precision_param in TORCH_DTYPE_NAMES
        assert self.training.mixed_precision_reduce in TORCH_DTYPE_NAMES
        assert self.training.fsdp_reshard_after_forward in {"default", "always", "never"}
        assert self.activation_checkpoint.mode in {"none", "selective", "full"}
        assert self.checkpoint.async_mode in {"disabled", "async", "async_with_pinned_mem"}
        assert self.lr_scheduler.decay_type in {"linear", "sqrt", "cosine"}
        self._refuse_unsupported()

    # Flags of the reference trainer that select machinery this framework does not have.  They parse (scripts that
    # pass their defaults keep working) but a non-default value is an error rather than a silent no-op.
    UNSUPPORTED = {
        "optimizer.early_step_in_backward": "the optimizer step runs after backward, fused with the parameter publication",
        "training.enable_cpu_offload": "optimizer state stays in device memory (180 GB per GPU)",
        "training.enable_expert_parallel": "no mixture-of-experts model is built",
        "training.compile": "there is no tracing compiler on the hot path; the fusions are hand-written kernels",
        "experimental.enable_compiled_autograd": "there is no tracing compiler on the hot path",
        "memory_estimation.enabled": "no fake-mode memory estimator is built",
        "fault_tolerance.enable": "replica-group fault tolerance (torchft) is not built",
        "float8.enable_fsdp_float8_all_gather": "float8 training is not built",
        "float8.precompute_float8_dynamic_scale_for_fsdp": "float8 training is not built",
        "float8.force_recompute_fp8_weight_in_bwd": "float8 training is not built",
        "float8.recipe_name": "float8 training is not built",
        "model.converters": "model converters (float8) are not built",
    }

    # Flags that pick, in the reference, another schedule of a computation this framework does one way; accepted (the
    # result is the same), with a note for the log.
    EQUIVALENT = {
        "optimizer.use_distributed_muon": "every Muon matrix is orthogonalised once, by its owner rank, and the update is "
                                          "published to the others (the reference's variant gathers the whole gradient on "
                                          "every rank and repeats the Newton-Schulz iteration there: same update)",
    }

    def equivalent_flag_notes(self) -> list[str]:
        """One line per accepted flag of ``EQUIVALENT`` that is set, for the trainer's start-up log."""
        notes = []
        for key, why in self.EQUIVALENT.items():
            section, name = key.split(".", 1)
            if getattr(getattr(self, section), name) not in (False, None, [], ""):
                notes.append(f"--{key}: {why}")
        return notes

    def _refuse_unsupported(self) -> None:
        for key, why in self.UNSUPPORTED.items():
            section, name = key.split(".", 1)
            value = getattr(getattr(self, section), name)
            if value not in (False, None, [], ""):
                raise NotImplementedError(f"--{key} is not supported: {why}")
