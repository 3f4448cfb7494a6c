"""Training data pipeline: online tokenisation into fixed-length windows, resumable shuffling,
collation (padded, stacked or packed variable-length) and a rank-aware stateful dataloader.

Covers the behaviour of the reference's flame/data.py: documents are tokenised in batches of 64,
concatenated and cut into ``seq_len`` windows with no document masking unless ``--training.varlen``
(157-211); the collator sets ``labels = input_ids.clone()`` — the shift happens inside the model —
and for packed batches derives ``cu_seqlens`` from BOS/EOS positions, splitting segments longer than
``context_len`` (311-498); dataloader state is stored per data-parallel rank (501-542);
``mds:/path?proc=glob&domain=a,b&seq_len=N`` selects pre-tokenised shards (567-572).
A ``synthetic:`` dataset (uniform random tokens) is added for benchmarking without any files.
"""
from __future__ import annotations

import pickle
from copy import deepcopy
from typing import Any, Iterable

import numpy as np
import torch
from torch.utils.data import IterableDataset

try:
    from torchdata.stateful_dataloader import StatefulDataLoader
except Exception:  # pragma: no cover
    from torch.utils.data import DataLoader as StatefulDataLoader


class SyntheticTokenDataset(IterableDataset):
    """Uniform random token windows: ``{'input_ids': LongTensor[seq_len]}``; resumable and rank-distinct."""

    def __init__(self, vocab_size: int, seq_len: int, rank: int = 0, world_size: int = 1, seed: int = 0):
        self.vocab_size, self.seq_len, self.rank, self.world_size, self.seed = vocab_size, seq_len, rank, world_size, seed
        self.index = 0

    def __iter__(self):
        while True:
            g = torch.Generator().manual_seed(self.seed * 1_000_003 + self.index * self.world_size + self.rank)
            self.index += 1
            yield {"input_ids": torch.randint(0, self.vocab_size, (self.seq_len,), generator=g, dtype=torch.long)}

    def state_dict(self):
        return {"index": self.index}

    def load_state_dict(self, sd):
        self.index = int(sd["index"])


class OnlineTokenizedIterableDataset(IterableDataset):
    """Tokenise a (sharded) text dataset on the fly and emit consecutive ``seq_len``-token windows."""

    DOCS_PER_CALL = 64

    def __init__(self, dataset, tokenizer, seq_len: int = 2048, rank: int = 0, world_size: int = 1, text_key: str | None = None):
        self.dataset, self.tokenizer, self.seq_len = dataset, tokenizer, seq_len
        self.rank, self.world_size, self.text_key = rank, world_size, text_key
        self.data = dataset.shard(world_size, rank) if hasattr(dataset, "shard") and world_size > 1 else dataset
        self.states = None          # state of the underlying HF iterable
        self.tokens: list[int] = []  # carry-over shorter than one window

    def _text(self, sample: dict) -> str:
        if self.text_key is not None:
            return sample[self.text_key]
        for key in ("text", "content"):
            if key in sample:
                return sample[key]
        raise KeyError(f"no text field in sample with keys {list(sample)}")

    def _encode(self, texts: list[str]) -> list[list[int]]:
        return self.tokenizer(texts, return_attention_mask=False)["input_ids"]

    def __iter__(self):
        if self.states is not None and hasattr(self.data, "load_state_dict"):
            self.data.load_state_dict(self.states)
        tokens = list(self.tokens)
        pending: list[str] = []
        states_before = self.data.state_dict() if hasattr(self.data, "state_dict") else None
        for sample in self.data:
            pending.append(self._text(sample))
            if len(pending) < self.DOCS_PER_CALL:
                continue
            for ids in self._encode(pending):
                tokens.extend(ids)
            pending = []
            states_after = self.data.state_dict() if hasattr(self.data, "state_dict") else None
            while len(tokens) >= self.seq_len:
                window, tokens = tokens[:self.seq_len], tokens[self.seq_len:]
                # resuming replays from the last fully consumed batch of documents
                self.states, self.tokens = (states_after if len(tokens) < self.seq_len else states_before), list(tokens)
                yield {"input_ids": torch.tensor(window, dtype=torch.long)}
            states_before = states_after
        if pending:
            for ids in self._encode(pending):
                tokens.extend(ids)
            while len(tokens) >= self.seq_len:
                window, tokens = tokens[:self.seq_len], tokens[self.seq_len:]
                self.tokens = list(tokens)
                yield {"input_ids": torch.tensor(window, dtype=torch.long)}

    def state_dict(self):
        return {"states": self.states, "tokens": list(self.tokens)}

    def load_state_dict(self, sd):
        self.states, self.tokens = sd.get("states"), list(sd.get("tokens", []))


class BufferShuffledIterableDataset(IterableDataset):
    """Reservoir-style shuffle buffer over another iterable dataset with a resumable RNG."""

    def __init__(self, dataset: Iterable, buffer_size: int = 1024, seed: int = 42):
        self.dataset, self.buffer_size, self.seed = dataset, buffer_size, seed
        self.rng_state = None
        self.buffer: list[Any] = []

    def __iter__(self):
        rng = np.random.default_rng(self.seed)
        if self.rng_state is not None:
            rng.bit_generator.state = self.rng_state
        buf = list(self.buffer)
        for item in self.dataset:
            if len(buf) < self.buffer_size:
                buf.append(item)
                continue
            i = int(rng.integers(0, self.buffer_size))
            out, buf[i] = buf[i], item
            self.rng_state, self.buffer = rng.bit_generator.state, buf
            yield out
        rng.shuffle(buf)
        while buf:
            out = buf.pop()
            self.buffer = buf
            yield out

    def state_dict(self):
        inner = self.dataset.state_dict() if hasattr(self.dataset, "state_dict") else None
        return {"rng": self.rng_state, "buffer": list(self.buffer), "inner": inner}

    def load_state_dict(self, sd):
        self.rng_state, self.buffer = sd.get("rng"), list(sd.get("buffer", []))
        if sd.get("inner") is not None and hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(sd["inner"])


class DataCollatorForLanguageModeling:
    """Batches ``{'input_ids': ...}`` samples.  ``labels`` is a clone of ``input_ids`` (padding -> -100)."""

    def __init__(self, tokenizer=None, context_len: int | None = None, varlen: bool = False, pad_token_id: int | None = None,
                 bos_token_id: int | None = None, eos_token_id: int | None = None):
        self.tokenizer, self.context_len, self.varlen = tokenizer, context_len, varlen
        tk = tokenizer
        self.pad_token_id = pad_token_id if pad_token_id is not None else getattr(tk, "pad_token_id", None)
        self.bos_token_id = bos_token_id if bos_token_id is not None else getattr(tk, "bos_token_id", None)
        self.eos_token_id = eos_token_id if eos_token_id is not None else getattr(tk, "eos_token_id", None)
        if varlen and self.bos_token_id is None and self.eos_token_id is None:
            raise ValueError("varlen packing needs a BOS or EOS token id to find document boundaries")

    def __call__(self, examples: list) -> dict[str, torch.Tensor]:
        ids = [torch.as_tensor(e["input_ids"] if isinstance(e, dict) else e, dtype=torch.long) for e in examples]
        if self.varlen:
            return self._packed(ids)
        same = all(t.numel() == ids[0].numel() for t in ids)
        if same:
            input_ids = torch.stack(ids)
            labels = input_ids.clone()
            return {"input_ids": input_ids, "labels": labels}
        if self.pad_token_id is None:
            raise ValueError("samples of different lengths need a pad token")
        width = max(t.numel() for t in ids)
        input_ids = torch.full((len(ids), width), self.pad_token_id, dtype=torch.long)
        mask = torch.zeros((len(ids), width), dtype=torch.long)
        for i, t in enumerate(ids):  # left padding keeps the last token aligned for generation
            input_ids[i, width - t.numel():] = t
            mask[i, width - t.numel():] = 1
        labels = input_ids.clone()
        labels[mask == 0] = -100
        return {"input_ids": input_ids, "labels": labels, "attention_mask": mask}

    def _packed(self, ids: list[torch.Tensor]) -> dict[str, torch.Tensor]:
        flat = torch.cat(ids).unsqueeze(0)
        total = flat.shape[1]
        if self.bos_token_id is not None:
            starts = (flat[0] == self.bos_token_id).nonzero().flatten()
        else:
            starts = (flat[0] == self.eos_token_id).nonzero().flatten() + 1
        bounds = torch.unique(torch.cat([torch.tensor([0]), starts, torch.tensor([total])]))
        bounds = bounds[bounds <= total]
        if self.context_len:
            pieces = [bounds[:1]]
            for a, b in zip(bounds[:-1].tolist(), bounds[1:].tolist()):
                pieces.append(torch.arange(a, b, self.context_len)[1:])
                pieces.append(torch.tensor([b]))
            bounds = torch.unique(torch.cat(pieces))
        return {"input_ids": flat, "labels": flat.clone(), "cu_seqlens": bounds.to(torch.int32)}


class ParallelAwareDataLoader(StatefulDataLoader):
    """Stateful dataloader whose state is keyed by the data-parallel rank that produced it."""

    def __init__(self, rank: int, dataset, batch_size: int, collate_fn, num_workers: int = 0, pin_memory: bool = False,
                 persistent_workers: bool = False, prefetch_factor: int | None = 2, snapshot_every_n_steps: int = 1):
        kwargs = dict(dataset=dataset, batch_size=batch_size, collate_fn=collate_fn, num_workers=num_workers,
                      pin_memory=pin_memory, persistent_workers=persistent_workers and num_workers > 0)
        if num_workers > 0:
            kwargs["prefetch_factor"] = prefetch_factor
        try:
            super().__init__(snapshot_every_n_steps=snapshot_every_n_steps, **kwargs)
        except TypeError:  # plain torch DataLoader fallback
            super().__init__(**kwargs)
        self.rank = rank

    def state_dict(self) -> dict[str, Any]:
        base = super().state_dict() if hasattr(super(), "state_dict") else {}
        return {f"rank_{self.rank}": pickle.dumps(base)}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        blob = state_dict.get(f"rank_{self.rank}")
        if blob is not None and hasattr(super(), "load_state_dict"):
            super().load_state_dict(pickle.loads(blob))


def _parse_probs(raw, n: int) -> list[float] | None:
    if raw is None:
        return None
    probs = [float(x) for x in str(raw).split(",")]
    if len(probs) != n:
        raise ValueError(f"data_probs has {len(probs)} entries for {n} datasets")
    total = sum(probs)
    return [p / total for p in probs]


def build_dataset(dataset: str, tokenizer, seq_len: int, rank: int, world_size: int, *, dataset_name=None,
                  dataset_split=None, data_dir=None, data_files=None, data_probs=None, streaming=True,
                  num_workers: int = 0, seed: int = 42, shuffle_buffer_size: int = 1024, vocab_size: int | None = None):
    """Dataset factory: ``synthetic:``, ``mds:``, or one / several HF datasets (comma separated)."""
    if dataset.startswith("synthetic"):
        v = vocab_size or getattr(tokenizer, "vocab_size", None) or 32000
        return SyntheticTokenDataset(v, seq_len, rank, world_size, seed)
    if dataset.startswith("mds:"):
        from .data_mds import build_mds_dataset
        return build_mds_dataset(dataset, seq_len=seq_len, rank=rank, world_size=world_size, seed=seed,
                                 shuffle=shuffle_buffer_size > 0)
    from datasets import interleave_datasets, load_dataset

    def split_arg(value, n):
        if value is None:
            return [None] * n
        parts = [p if p not in ("", "None") else None for p in str(value).split(",")]
        return parts * n if len(parts) == 1 else parts

    names = dataset.split(",")
    n = len(names)
    subsets, splits, dirs, files = (split_arg(v, n) for v in (dataset_name, dataset_split, data_dir, data_files))
    loaded = []
    for i, name in enumerate(names):
        ds = load_dataset(path=name, name=subsets[i], split=splits[i] or "train", data_dir=dirs[i], data_files=files[i],
                          streaming=streaming, trust_remote_code=True)
        min_shards = world_size * max(1, num_workers)
        if hasattr(ds, "num_shards") and ds.num_shards < min_shards and not streaming:
            ds = ds.to_iterable_dataset(num_shards=min_shards)
        if shuffle_buffer_size > 0 and hasattr(ds, "shuffle"):
            ds = ds.shuffle(seed=seed, buffer_size=shuffle_buffer_size) if streaming else ds.shuffle(seed=seed)
        loaded.append(ds)
    if n == 1:
        merged = loaded[0]
    else:
        merged = interleave_datasets(loaded, probabilities=_parse_probs(data_probs, n), seed=seed,
                                     stopping_strategy="all_exhausted")
    return OnlineTokenizedIterableDataset(merged, tokenizer, seq_len, rank, world_size)


def build_dataloader(dataset, tokenizer, rank: int, batch_size: int, *, context_len=None, varlen=False, num_workers=0,
                     pin_memory=False, persistent_workers=False, prefetch_factor=2, snapshot_every_n_steps=1,
                     pad_token_id=None, bos_token_id=None, eos_token_id=None):
    collate = DataCollatorForLanguageModeling(tokenizer, context_len, varlen, pad_token_id, bos_token_id, eos_token_id)
    return ParallelAwareDataLoader(rank, dataset, batch_size, collate, num_workers, pin_memory, persistent_workers,
                                   prefetch_factor, snapshot_every_n_steps)
