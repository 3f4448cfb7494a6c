"""Checkpointing in the reference's ``torch.distributed.checkpoint`` (DCP) layout.

A checkpoint is the directory ``{dump_folder}/{folder}/step-{N}`` holding ``.metadata`` and
``__{rank}_{i}.distcp`` files.  Training checkpoints nest everything under top-level names, so model
tensors appear as ``model.<param name>`` (``model.model.embeddings.weight``); converter output and seed
checkpoints hold raw parameter names.  Both conventions load (scripts/eval_token_ppl.py:75-92 and
flame/utils/convert_dcp_to_hf.py:57 in the reference rely on this).  Optimizer state is saved as full
per-parameter fp32 tensors gathered from the shards, so a run can resume on a different number of
GPUs.  ``TrainState`` mirrors flame/components/checkpoint.py:21-58.
"""
from __future__ import annotations

import os
import pickle
import re
import shutil
import threading
import time
from dataclasses import dataclass, field
from io import BytesIO
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.stateful import Stateful

_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


@dataclass
class TrainState(Stateful):
    step: int = 0
    skipped_step: int = 0
    token: int = 0
    elapsed: float = 0.0
    global_avg_losses: list[float] = field(default_factory=list)
    global_max_losses: list[float] = field(default_factory=list)
    log_steps: list[int] = field(default_factory=list)

    @staticmethod
    def _pack(obj) -> BytesIO:
        buf = BytesIO()
        torch.save(obj, buf)
        return buf

    def state_dict(self) -> dict[str, Any]:
        return {
            "step": torch.tensor(self.step, dtype=torch.int32),
            "skipped_step": torch.tensor(self.skipped_step, dtype=torch.int32),
            "token": torch.tensor(self.token, dtype=torch.int64),
            "elapsed": torch.tensor(self.elapsed, dtype=torch.float64),
            "global_avg_losses": self._pack(self.global_avg_losses),
            "global_max_losses": self._pack(self.global_max_losses),
            "log_steps": self._pack(self.log_steps),
        }

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.step = int(sd["step"])
        self.skipped_step = int(sd.get("skipped_step", 0))
        self.token = int(sd["token"])
        self.elapsed = float(sd["elapsed"])
        for name in ("global_avg_losses", "global_max_losses", "log_steps"):
            buf = sd[name]
            buf.seek(0)
            setattr(self, name, torch.load(buf, weights_only=False))


def checkpoint_keys(path: str) -> set[str]:
    """Names of the tensors/objects stored in a DCP directory."""
    reader = dcp.FileSystemReader(path)
    return set(reader.read_metadata().state_dict_metadata.keys())


def detect_model_prefix(keys: set[str]) -> str:
    """'model.' for training checkpoints (nested under "model"), '' for raw converter output."""
    if any(k.startswith("model.model.") or k.startswith("model.lm_head.") for k in keys):
        return "model."
    return ""


def load_model_weights(model: torch.nn.Module, path: str, exclude: list[str] | None = None, strict: bool = False,
                       loaded: dict[int, torch.Tensor] | None = None) -> list[str]:
    """Load model tensors from a DCP directory of either key convention.  Returns missing names.

    Tensors are read in the dtype they were saved in and cast on the copy into the model; ``loaded`` (if given)
    receives ``{parameter data_ptr: tensor as saved}`` so that a caller holding fp32 master weights can take the
    full-precision values instead of the rounded ones."""
    reader = dcp.FileSystemReader(path)
    meta = reader.read_metadata().state_dict_metadata
    keys = set(meta.keys())
    prefix = detect_model_prefix(keys)
    own = model.state_dict()
    exclude = exclude or []
    wanted, missing = {}, []
    seen_ptr: dict[int, str] = {}
    tp = getattr(model, "_tp", None)          # tensor parallel: checkpoints hold full tensors, ranks keep slices
    params = dict(model.named_parameters()) if tp is not None else {}
    for name, tensor in own.items():
        if any(name.startswith(e) for e in exclude):
            continue
        if prefix + name in keys:
            props = getattr(meta[prefix + name], "properties", None)
            saved_dtype = getattr(props, "dtype", None) or tensor.dtype
            if tp is not None and name in params:
                from ..parallel.tensor import full_shape
                wanted[prefix + name] = torch.empty(full_shape(params[name]), dtype=saved_dtype, device="cpu")
                continue
            wanted[prefix + name] = torch.empty(tensor.shape, dtype=saved_dtype, device="cpu")
        else:
            missing.append(name)
    dcp.load(wanted, checkpoint_id=path, no_dist=not (dist.is_available() and dist.is_initialized()))
    with torch.no_grad():
        for key, value in wanted.items():
            name = key[len(prefix):]
            ptr = own[name].data_ptr()
            if ptr in seen_ptr:          # tied tensors: the first name wins
                continue
            seen_ptr[ptr] = name
            if tp is not None:
                from ..parallel.tensor import slice_named
                value = slice_named(model, tp, {name: value})[name]
            own[name].copy_(value.to(own[name].dtype))
            if loaded is not None:
                loaded[ptr] = value
    tied_ok = {"lm_head.weight", "model.embeddings.weight"}
    hard_missing = [m for m in missing if m not in tied_ok and "rotary" not in m]
    if strict and hard_missing:
        raise KeyError(f"missing keys in {path}: {hard_missing[:8]}")
    return missing


class CheckpointManager:
    """Save / load / purge policy of the trainer (interval, last step, external trigger, keep_latest_k)."""

    def __init__(self, engine, train_state: TrainState, job_config, dataloader=None, lr_state=None, logger=None):
        ck = job_config.checkpoint
        self.engine, self.train_state, self.dataloader, self.lr_state = engine, train_state, dataloader, lr_state
        self.enable = bool(ck.enable_checkpoint)
        self.folder = os.path.join(job_config.job.dump_folder, ck.folder)
        self.initial_load_path = ck.initial_load_path
        self.initial_weights_only = bool(ck.initial_load_model_weights_only)
        self.interval = int(ck.interval)
        self.last_weights_only = bool(ck.last_save_model_weights_only)
        self.export_dtype = _DTYPES[ck.export_dtype]
        self.keep_latest_k = int(ck.keep_latest_k)
        self.load_step = int(ck.load_step)
        self.exclude = list(ck.exclude_from_loading or [])
        self.async_mode = ck.async_mode
        self.logger = logger
        self._async_future = None
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1

    # ------------------------------------------------------------------------------ helpers
    def _log(self, msg: str):
        if self.logger:
            self.logger.info(msg)

    def _step_dir(self, step: int) -> str:
        return os.path.join(self.folder, f"step-{step}")

    def available_steps(self) -> list[int]:
        if not os.path.isdir(self.folder):
            return []
        steps = []
        for name in os.listdir(self.folder):
            m = re.fullmatch(r"step-(\d+)", name)
            if m and os.path.isfile(os.path.join(self.folder, name, ".metadata")):
                steps.append(int(m.group(1)))
        return sorted(steps)

    def _model_state(self, dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
        """Full-precision model tensors rebuilt from the fp32 master shards (tied weights written twice)."""
        out = {}
        with self.engine.sdp.full_parameters():        # sharded weights: every parameter addressable (and distinct) in full
            full = self.engine.sdp.gather_full("master")
            for name, p in self.engine.model.state_dict().items():
                src = full.get(p.data_ptr())
                t = src if src is not None else p.detach().float().clone()
                out[name] = t.to(dtype) if dtype is not None else t
        tp = getattr(self.engine, "tp", None)
        if tp is not None:
            from ..parallel.tensor import gather_named
            out = gather_named(self.engine.model, tp, out)
        return out

    def _states(self, model_only: bool, dtype=None) -> dict[str, Any]:
        if model_only:
            return self._model_state(dtype)          # raw keys: loadable as a seed / by converters
        sd: dict[str, Any] = {"model": self._model_state(None)}
        sd["optimizer"] = self.engine.sdp.full_optimizer_state()
        if getattr(self.engine, "tp", None) is not None:
            from ..parallel.tensor import gather_named
            sd["optimizer"] = gather_named(self.engine.model, self.engine.tp, sd["optimizer"])
        sd["train_state"] = self.train_state.state_dict()
        if self.lr_state is not None:
            sd["lr_scheduler"] = {"last_step": torch.tensor(int(self.lr_state()), dtype=torch.int64)}
        if self.dataloader is not None and hasattr(self.dataloader, "state_dict"):
            sd["dataloader"] = {f"rank_{self.rank}": self._bytes(self.dataloader.state_dict())}
        return sd

    @staticmethod
    def _bytes(obj) -> BytesIO:
        buf = BytesIO()
        pickle.dump(obj, buf)
        buf.seek(0)
        return buf

    # ------------------------------------------------------------------------------ save
    def should_save(self, step: int, last: bool = False, force: bool = False) -> bool:
        if not self.enable:
            return False
        return force or last or (self.interval > 0 and step % self.interval == 0)

    def maybe_wait_for_staging(self):
        if self._async_future is not None:
            self._async_future.result()
            self._async_future = None

    def save(self, step: int, last: bool = False, force: bool = False) -> bool:
        if not self.should_save(step, last, force):
            return False
        self.maybe_wait_for_staging()
        t0 = time.perf_counter()
        model_only = last and self.last_weights_only
        state = self._states(model_only, self.export_dtype if model_only else None)
        path = self._step_dir(step)
        if self.async_mode != "disabled" and not last:
            cpu_state = _to_cpu(state)
            self._async_future = dcp.async_save(cpu_state, checkpoint_id=path)
        else:
            dcp.save(state, checkpoint_id=path, no_dist=self.world == 1)
        self._log(f"saved checkpoint step-{step} ({'weights only' if model_only else 'full'}) in {time.perf_counter() - t0:.1f}s")
        self._purge()
        return True

    def save_seed(self):
        dcp.save(self._model_state(None), checkpoint_id=self._step_dir(0), no_dist=self.world == 1)

    def _purge(self):
        if self.keep_latest_k <= 0 or self.rank != 0:
            return
        steps = self.available_steps()
        doomed = steps[:-self.keep_latest_k]
        if doomed:
            threading.Thread(target=lambda: [shutil.rmtree(self._step_dir(s), ignore_errors=True) for s in doomed],
                             daemon=True).start()

    # ------------------------------------------------------------------------------ load
    def load(self, step: int = -1) -> bool:
        """Resume from ``folder`` (newest or ``step``); else start from ``initial_load_path``."""
        if not self.enable and not self.initial_load_path:
            return False
        steps = self.available_steps()
        if steps:
            step = self.load_step if self.load_step >= 0 else (steps[-1] if step < 0 else step)
            if step not in steps:
                raise FileNotFoundError(f"no checkpoint step-{step} under {self.folder}")
            path = self._step_dir(step)
            weights_only = step == 0
        elif self.initial_load_path:
            path, weights_only = self.initial_load_path, self.initial_weights_only
        else:
            return False
        t0 = time.perf_counter()
        try:
            as_saved: dict[int, torch.Tensor] = {}
            with self.engine.sdp.full_parameters():
                load_model_weights(self.engine.model, path, self.exclude, loaded=as_saved)
                self.engine.sdp.resync_master()
                # checkpoints written by this trainer hold the fp32 masters: take them as they are, so that a resumed
                # run continues from exactly the weights the interrupted one had (not from their bf16 rounding)
                self.engine.sdp.load_full_master(as_saved)
            keys = checkpoint_keys(path)
            if not weights_only and any(k.startswith("optimizer.") for k in keys):
                self._load_training_state(path, keys)
        except dcp.api.CheckpointException as exc:      # derives from BaseException: turn it into a normal error
            older = [s for s in steps if s < step] if steps else []
            hint = f"; resume from an older one with --checkpoint.load_step {older[-1]}" if older else ""
            raise RuntimeError(f"checkpoint {path} is unreadable (truncated or corrupted shard){hint}") from exc
        self._log(f"loaded checkpoint {path} in {time.perf_counter() - t0:.1f}s")
        return True

    def _load_training_state(self, path: str, keys: set[str]):
        no_dist = self.world == 1
        opt_template = {"optimizer": self.engine.sdp.full_optimizer_state(template=True)}
        tp = getattr(self.engine, "tp", None)
        if tp is not None:      # saved states of sharded weights have the full shape
            from ..parallel.tensor import _shard_spec, slice_named
            for key, t in list(opt_template["optimizer"].items()):
                spec = _shard_spec(self.engine.model, key) if isinstance(t, torch.Tensor) and t.dim() > 0 else None
                if spec is not None:
                    shape = list(t.shape)
                    shape[spec[0]] *= spec[1]
                    opt_template["optimizer"][key] = torch.empty(shape, dtype=t.dtype, device=t.device)
        dcp.load(opt_template, checkpoint_id=path, no_dist=no_dist)
        if tp is not None:
            opt_template["optimizer"] = slice_named(self.engine.model, tp, opt_template["optimizer"])
        self.engine.sdp.load_full_optimizer_state(opt_template["optimizer"])
        ts = {"train_state": self.train_state.state_dict()}
        dcp.load(ts, checkpoint_id=path, no_dist=no_dist)
        self.train_state.load_state_dict(ts["train_state"])
        dl_key = f"dataloader.rank_{self.rank}"
        if self.dataloader is not None and dl_key in keys and hasattr(self.dataloader, "load_state_dict"):
            dl = {"dataloader": {f"rank_{self.rank}": BytesIO()}}
            dcp.load(dl, checkpoint_id=path, no_dist=no_dist)
            buf = dl["dataloader"][f"rank_{self.rank}"]
            buf.seek(0)
            self.dataloader.load_state_dict(pickle.load(buf))


def _to_cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    return obj
