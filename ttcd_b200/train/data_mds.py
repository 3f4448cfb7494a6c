"""Pre-tokenised MDS shards: ``mds:/path?proc=glob&domain=a,b&seq_len=N``.

Same URI grammar, directory discovery (``root/<domain>/<proc*-64>/``) and sample contract
(``{'input_ids': LongTensor[seq_len]}``, longer samples truncated) as the reference dataset
(flame/data_mds.py:39-48, 51-67, 70-125, 128-141).  The reference delegates shard reading, shuffling and
data-parallel sharding to the mosaicml-streaming package; that package is not a dependency here.  This
module reads the (uncompressed) MDS shard format itself through ``numpy.memmap`` — the samples of a 64K
recipe are 256 KiB each, so a memory-mapped read straight into the pinned staging buffer is the cheapest
path to the GPU — and does its own seeded, resumable, rank-strided shuffling.

Shard layout (little endian): ``uint32 n`` | ``uint32 offsets[n+1]`` (byte offsets from the file start) |
``n`` samples.  A sample holds, for the columns of ``index.json`` in order, first one ``uint32`` size for
every variable-size column, then the column payloads.  Supported encodings: ``bytes``, ``str``, ``int``,
``uint8..int64``, ``float32/64`` scalars and ``ndarray[:dtype[:shape]]``.
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass

import numpy as np
import torch
from torch.utils.data import IterableDataset

_SCALARS = {"int": np.int64, "uint8": np.uint8, "uint16": np.uint16, "uint32": np.uint32, "uint64": np.uint64,
            "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64, "float16": np.float16,
            "float32": np.float32, "float64": np.float64}


def parse_mds_uri(uri: str) -> tuple[str, dict]:
    if not uri.startswith("mds:"):
        raise ValueError(f"not an mds: URI: {uri!r}")
    body = uri[4:]
    path, _, query = body.partition("?")
    params = dict(pair.split("=", 1) for pair in query.split("&") if pair)
    return path, params


def discover_proc_dirs(root: str, proc_glob: str | None = None, domain_filter: set[str] | None = None) -> list[str]:
    proc_glob = proc_glob or "proc*-64"
    found = []
    for domain in sorted(os.listdir(root)):
        full = os.path.join(root, domain)
        if domain.startswith(".") or not os.path.isdir(full):
            continue
        if domain_filter is not None and domain not in domain_filter:
            continue
        found += [p for p in sorted(glob.glob(os.path.join(full, proc_glob))) if os.path.isdir(p)]
    return found


# --------------------------------------------------------------------------------------- shard format
def _decode_ndarray(encoding: str, raw: np.ndarray) -> np.ndarray:
    parts = encoding.split(":")
    if len(parts) >= 2:                                    # dtype fixed by the index
        dtype = np.dtype(parts[1])
        if len(parts) == 3:                                # shape fixed as well: payload is the data only
            shape = tuple(int(s) for s in parts[2].split(","))
            return raw.view(dtype).reshape(shape)
        ndim = int(raw[0])                                 # uint8 ndim, then uint32 dims... (dynamic shape)
        shape = raw[1:1 + 4 * ndim].view(np.uint32)
        return raw[1 + 4 * ndim:].view(dtype).reshape(tuple(int(s) for s in shape))
    # fully dynamic: uint8 dtype code, uint8 ndim, uint32 dims, data
    codes = [np.uint8, np.int8, np.uint16, np.int16, np.uint32, np.int32, np.uint64, np.int64, np.float16, np.float32,
             np.float64]
    dtype = np.dtype(codes[int(raw[0])])
    ndim = int(raw[1])
    shape = raw[2:2 + 4 * ndim].view(np.uint32)
    return raw[2 + 4 * ndim:].view(dtype).reshape(tuple(int(s) for s in shape))


@dataclass
class _Shard:
    path: str
    samples: int
    names: list[str]
    encodings: list[str]
    sizes: list[int | None]
    _map: np.ndarray | None = None
    _offsets: np.ndarray | None = None

    def _open(self):
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="r")
            n = int(self._map[:4].view(np.uint32)[0])
            if n != self.samples:
                raise ValueError(f"{self.path}: header says {n} samples, index says {self.samples}")
            self._offsets = np.asarray(self._map[4:4 + 4 * (n + 1)].view(np.uint32))

    def sample(self, i: int, only: str | None = None) -> dict:
        self._open()
        raw = self._map[int(self._offsets[i]):int(self._offsets[i + 1])]
        nvar = sum(1 for s in self.sizes if s is None)
        var_sizes = iter(raw[:4 * nvar].view(np.uint32).tolist())
        pos = 4 * nvar
        out = {}
        for name, enc, size in zip(self.names, self.encodings, self.sizes):
            size = next(var_sizes) if size is None else size
            field = raw[pos:pos + size]
            pos += size
            if only is not None and name != only:
                continue
            if enc == "bytes":
                out[name] = bytes(field)
            elif enc == "str":
                out[name] = bytes(field).decode("utf-8")
            elif enc in _SCALARS:
                out[name] = field.view(_SCALARS[enc])[0].item()
            elif enc.startswith("ndarray"):
                out[name] = _decode_ndarray(enc, field)
            else:
                raise NotImplementedError(f"MDS column encoding {enc!r}")
        return out


def read_index(directory: str) -> list[_Shard]:
    with open(os.path.join(directory, "index.json")) as f:
        index = json.load(f)
    shards = []
    for entry in index["shards"]:
        if entry.get("format", "mds") != "mds":
            raise NotImplementedError(f"shard format {entry.get('format')!r}")
        if entry.get("compression"):
            raise NotImplementedError("compressed MDS shards are not supported; decompress them first")
        shards.append(_Shard(os.path.join(directory, entry["raw_data"]["basename"]), int(entry["samples"]),
                             list(entry["column_names"]), list(entry["column_encodings"]), list(entry["column_sizes"])))
    return shards


def write_mds(directory: str, samples: list[dict], columns: dict[str, str], shard_samples: int = 1 << 30) -> None:
    """Write samples as uncompressed MDS shards (used by tests and by offline pre-tokenisation)."""
    os.makedirs(directory, exist_ok=True)
    names = sorted(columns)
    encs = [columns[n] for n in names]

    def fixed(enc: str):
        if enc in _SCALARS:
            return np.dtype(_SCALARS[enc]).itemsize
        p = enc.split(":")
        if p[0] == "ndarray" and len(p) == 3:
            return int(np.prod([int(s) for s in p[2].split(",")])) * np.dtype(p[1]).itemsize
        return None

    sizes = [fixed(e) for e in encs]

    def encode(enc: str, value) -> bytes:
        if enc == "bytes":
            return bytes(value)
        if enc == "str":
            return value.encode("utf-8")
        if enc in _SCALARS:
            return np.asarray(value, dtype=_SCALARS[enc]).tobytes()
        p = enc.split(":")
        arr = np.asarray(value)
        if len(p) == 3:
            return arr.astype(p[1]).tobytes()
        if len(p) == 2:
            arr = arr.astype(p[1])
            return bytes([arr.ndim]) + np.asarray(arr.shape, dtype=np.uint32).tobytes() + arr.tobytes()
        raise NotImplementedError(enc)

    entries = []
    for s0 in range(0, len(samples), shard_samples):
        chunk = samples[s0:s0 + shard_samples]
        blobs = []
        for smp in chunk:
            fields = [encode(e, smp[n]) for n, e in zip(names, encs)]
            head = b"".join(np.uint32(len(f)).tobytes() for f, sz in zip(fields, sizes) if sz is None)
            blobs.append(head + b"".join(fields))
        n = len(blobs)
        offsets = np.zeros(n + 1, dtype=np.uint32)
        offsets[0] = 4 + 4 * (n + 1)
        offsets[1:] = offsets[0] + np.cumsum([len(b) for b in blobs], dtype=np.uint64).astype(np.uint32)
        base = f"shard.{len(entries):05d}.mds"
        with open(os.path.join(directory, base), "wb") as f:
            f.write(np.uint32(n).tobytes() + offsets.tobytes() + b"".join(blobs))
        entries.append({"format": "mds", "compression": None, "samples": n, "column_names": names, "column_encodings": encs,
                        "column_sizes": sizes, "raw_data": {"basename": base, "bytes": int(offsets[-1]), "hashes": {}},
                        "hashes": [], "size_limit": None, "version": 2, "zip_data": None})
    with open(os.path.join(directory, "index.json"), "w") as f:
        json.dump({"version": 2, "shards": entries}, f)


# --------------------------------------------------------------------------------------- dataset
class MDSPretokenizedDataset(IterableDataset):
    """All samples of all matching ``proc`` directories, shuffled with a seeded permutation per epoch and
    dealt ``rank::world_size`` (then ``worker::num_workers``).  ``state_dict`` / ``load_state_dict`` resume
    exactly (epoch + position)."""

    def __init__(self, root: str, seq_len: int = 65536, proc_glob: str | None = "proc0[0-9]-64",
                 domain_filter: set[str] | None = None, shuffle: bool = True, seed: int = 42, rank: int = 0,
                 world_size: int = 1):
        dirs = discover_proc_dirs(root, proc_glob, domain_filter)
        if not dirs and os.path.isfile(os.path.join(root, "index.json")):
            dirs = [root]                                   # a single stream directory is accepted as well
        if not dirs:
            raise FileNotFoundError(f"No MDS proc dirs under {root} matching glob={proc_glob!r}, domain_filter={domain_filter}")
        self.seq_len, self.shuffle, self.seed, self.rank, self.world_size = seq_len, shuffle, seed, rank, world_size
        self.shards = [s for d in dirs for s in read_index(d)]
        self.cum = np.cumsum([0] + [s.samples for s in self.shards])
        self.epoch, self.position = 0, 0

    def __len__(self):
        return int(self.cum[-1])

    def _order(self, epoch: int) -> np.ndarray:
        n = len(self)
        if not self.shuffle:
            return np.arange(n)
        return np.random.default_rng([self.seed, epoch]).permutation(n)

    def get(self, index: int) -> torch.Tensor:
        s = int(np.searchsorted(self.cum, index, side="right")) - 1
        ids = self.shards[s].sample(index - int(self.cum[s]), only="input_ids")["input_ids"]
        ids = np.frombuffer(ids, dtype=np.int32) if isinstance(ids, bytes) else ids
        return torch.from_numpy(np.ascontiguousarray(ids[:self.seq_len]).astype(np.int64))

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        wid, nworkers = (info.id, info.num_workers) if info is not None else (0, 1)
        stride = self.world_size * nworkers
        first = self.rank * nworkers + wid
        while True:
            order = self._order(self.epoch)
            mine = order[first::stride]
            while self.position < len(mine):
                idx = int(mine[self.position])
                self.position += 1
                yield {"input_ids": self.get(idx)}
            self.epoch += 1
            self.position = 0

    def state_dict(self):
        return {"epoch": self.epoch, "position": self.position}

    def load_state_dict(self, state):
        self.epoch, self.position = int(state["epoch"]), int(state["position"])


def build_mds_dataset(uri: str, seq_len: int | None = None, seed: int = 42, *, rank: int = 0, world_size: int = 1,
                      default_seq_len: int = 65536, shuffle: bool = True) -> MDSPretokenizedDataset:
    path, params = parse_mds_uri(uri)
    domain_filter = set(params["domain"].split(",")) if "domain" in params else None
    return MDSPretokenizedDataset(path, seq_len=int(params.get("seq_len", seq_len or default_seq_len)),
                                  proc_glob=params.get("proc", "proc0[0-9]-64"), domain_filter=domain_filter,
                                  shuffle=shuffle, seed=seed, rank=rank, world_size=world_size)
