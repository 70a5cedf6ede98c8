"""A reader for GGUF files: metadata and plain (unquantized) tensors.

The reference reads nothing but GGUF (gguf/src/lib.rs:21-126): it maps the file, parses the key-value
metadata and the tensor table, and hands out byte slices by tensor name.  This reader does the same
for the value types the architecture's keys use and the tensor types the engine takes: F32, F16
and BF16.  Quantized tensor types are recognised by number and refused by the loader with their name.

A model may be cut into shards ``<name>-0000N-of-0000M.gguf``: given the path of ANY shard,
:func:`open_gguf` maps all M of them and merges their metadata and tensor tables, as the reference does
(gguf/src/lib.rs:21-48 maps the shards, :76-126 merges them): ``general.alignment`` and ``split.*`` keys
are every shard's own and are left out; any other metadata key, or a tensor name, that appears in two
shards is an error.

Layout (version 2 and 3, little endian):
    magic "GGUF" | version u32 | tensor count u64 | metadata count u64
    metadata: key (u64 length + bytes) | value type u32 | value
    tensor table: name | n_dims u32 | dims u64 x n_dims (innermost first) | type u32 | offset u64
    padding to ``general.alignment`` (default 32) | tensor data
"""
from __future__ import annotations

import mmap
import os
import re
import struct
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Tuple

import numpy as np
import torch


class GGufError(ValueError):
    pass


_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9
# ggml tensor types the engine can take, and the names of some it cannot (for the error message)
_PLAIN = {0: ("F32", np.dtype("<f4"), torch.float32), 1: ("F16", np.dtype("<f2"), torch.float16),
          30: ("BF16", np.dtype("<u2"), torch.bfloat16)}
_OTHER = {2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K",
          13: "Q5_K", 14: "Q6_K", 15: "Q8_K", 24: "I8", 25: "I16", 26: "I32", 27: "I64", 28: "F64"}


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGufError("the file ends inside its header")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GGufError("the file ends inside a string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, t):
        if t in _SCALARS:
            return self.take(_SCALARS[t])
        if t == _STRING:
            return self.string()
        if t == _ARRAY:
            et, n = self.take("<I"), self.take("<Q")
            if et in _SCALARS and et != 7:
                fmt = np.dtype(_SCALARS[et])
                size = fmt.itemsize * n
                if self.pos + size > len(self.buf):
                    raise GGufError("the file ends inside an array")
                arr = np.frombuffer(self.buf, dtype=fmt, count=n, offset=self.pos).tolist()
                self.pos += size
                return arr
            return [self.value(et) for _ in range(n)]
        raise GGufError(f"unknown metadata value type {t}")


class GGufFile:
    """metadata: {key: value}; tensors: {name: (shape row-major, ggml type number, byte offset in the file)}."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        try:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:
            raise GGufError(f"{path} is empty") from None
        r = _Reader(self._map)
        if bytes(self._map[:4]) != b"GGUF":
            raise GGufError(f"{path} is not a GGUF file (bad magic)")
        r.pos = 4
        self.version = r.take("<I")
        if self.version not in (2, 3):
            raise GGufError(f"GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = r.string()
            if key in self.metadata:
                raise GGufError(f"metadata key {key!r} appears twice")      # gguf/src/lib.rs:99-110
            self.metadata[key] = r.value(r.take("<I"))
        infos = []
        for _ in range(n_tensors):
            name = r.string()
            nd = r.take("<I")
            dims = [r.take("<Q") for _ in range(nd)]
            infos.append((name, tuple(reversed(dims)), r.take("<I"), r.take("<Q")))
        align = int(self.metadata.get("general.alignment", 32))
        data0 = (r.pos + align - 1) // align * align
        self.tensors: Dict[str, Tuple[Tuple[int, ...], int, int]] = {}
        for name, shape, t, off in infos:
            if name in self.tensors:
                raise GGufError(f"tensor {name!r} appears twice")           # gguf/src/lib.rs:112-124
            self.tensors[name] = (shape, t, data0 + off)
        for name, (shape, t, off) in self.tensors.items():
            if t in _PLAIN and off + int(np.prod(shape, dtype=np.int64)) * _PLAIN[t][1].itemsize > len(self._map):
                raise GGufError(f"tensor {name!r} reaches beyond the end of the file (truncated?)")

    # ---- the interface the weight loader uses ---------------------------------------------------
    def names(self):
        return self.tensors.keys()

    def shape_dtype(self, name: str):
        shape, t, _ = self.tensors[name]
        return shape, (_PLAIN[t][0] if t in _PLAIN else _OTHER.get(t, f"GGML_TYPE_{t}"))

    def tensor(self, name: str) -> torch.Tensor:
        shape, t, off = self.tensors[name]
        if t not in _PLAIN:
            raise GGufError(f"tensor {name!r} has type {self.shape_dtype(name)[1]}: quantized tensors are not supported")
        _, npdt, tdt = _PLAIN[t]
        n = int(np.prod(shape, dtype=np.int64))
        arr = np.frombuffer(self._map, dtype=npdt, count=n, offset=off).reshape(shape)
        out = torch.from_numpy(arr.copy())
        return out.view(torch.bfloat16) if tdt == torch.bfloat16 else out

    def config(self) -> dict:
        return config_of(self.metadata, self.tensors)


def config_of(metadata: Dict[str, Any], tensors: Dict[str, Tuple]) -> dict:
    """The metadata as a configuration dict: the architecture's own keys as they are, plus the
    vocabulary size the way the reference finds it (the length of ``tokenizer.ggml.tokens``,
    models/llama/common/src/storage.rs:48) or, failing that, the rows of ``token_embd.weight``."""
    cfg = {k: v for k, v in metadata.items() if not isinstance(v, list) or len(v) <= 16}
    arch = metadata.get("general.architecture")
    if arch and f"{arch}.vocab_size" not in cfg:
        toks = metadata.get("tokenizer.ggml.tokens")
        if isinstance(toks, list):
            cfg[f"{arch}.vocab_size"] = len(toks)
        elif "token_embd.weight" in tensors:
            cfg[f"{arch}.vocab_size"] = tensors["token_embd.weight"][0][0]
    if "output.weight" not in tensors:
        cfg.setdefault("tie_word_embeddings", True)                      # storage.rs:84
    return cfg


_SHARD = re.compile(r"^(?P<stem>.*)-(?P<n>\d{5})-of-(?P<m>\d{5})\.gguf$")


def shard_paths(path: str) -> List[str]:
    """All shards of the model that ``path`` is one shard of, in order; [path] for a file that is whole."""
    folder, name = os.path.split(path)
    m = _SHARD.match(name)
    if m is None or int(m["m"]) <= 1:
        return [path]
    count = int(m["m"])
    if not (1 <= int(m["n"]) <= count):
        raise GGufError(f"{name}: shard number {int(m['n'])} lies outside 1..{count}")
    return [os.path.join(folder, f"{m['stem']}-{i:05d}-of-{count:05d}.gguf") for i in range(1, count + 1)]


class GGufModel:
    """A model from several shard files, behind the interface of :class:`GGufFile`."""

    def __init__(self, paths: List[str]):
        missing = [p for p in paths if not os.path.isfile(p)]
        if missing:
            raise GGufError(f"shards missing: {', '.join(os.path.basename(p) for p in missing)} "
                            f"(of {len(paths)} in {os.path.dirname(paths[0]) or '.'})")
        self.path = paths[0]
        with ThreadPoolExecutor(max_workers=min(8, len(paths))) as pool:     # a thread per shard, gguf/src/lib.rs:82-96
            self.shards = list(pool.map(GGufFile, paths))
        self.metadata: Dict[str, Any] = {}
        self.tensors: Dict[str, Tuple] = {}
        self._where: Dict[str, GGufFile] = {}
        for i, f in enumerate(self.shards):
            for k, v in f.metadata.items():
                if k == "general.alignment" or k.startswith("split."):
                    continue                                                     # gguf/src/lib.rs:101-103
                if k in self.metadata:
                    raise GGufError(f"shard {i + 1} ({os.path.basename(f.path)}): metadata key {k!r} is in an earlier "
                                    f"shard too")
                self.metadata[k] = v
            for name, info in f.tensors.items():
                if name in self.tensors:
                    raise GGufError(f"shard {i + 1} ({os.path.basename(f.path)}): tensor {name!r} is in an earlier "
                                    f"shard too")
                self.tensors[name] = info
                self._where[name] = f

    def names(self):
        return self.tensors.keys()

    def shape_dtype(self, name: str):
        return self._where[name].shape_dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def config(self) -> dict:
        return config_of(self.metadata, self.tensors)


def open_gguf(path: str):
    """The model that ``path`` belongs to: one file, or all shards of a sharded one."""
    paths = shard_paths(path)
    return GGufFile(path) if len(paths) == 1 else GGufModel(paths)
