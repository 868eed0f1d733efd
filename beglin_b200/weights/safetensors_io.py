"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the tensors' bytes (safetensors_load.h:5-13).

The reader checks what the reference's reader checks before it trusts a file: the header fits in
the file (safetensors_load.c:210-214), every tensor has dtype, shape and offsets (:249-252), at
most 8 dimensions (:253-257), offsets ordered and inside the data section (:258-263), a known dtype
(:268-271), and a byte count that equals the shape's.  A folder is read through `model.safetensors`
or, when that is absent, through `model.safetensors.index.json` and the shards its `weight_map`
names, whose file names must be plain base names (:338, :346-419).

Tensors keep the type they are stored in: BF16 stays bfloat16, F32 stays float32, F16 stays float16;
integer tables come back as int32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    # name: (bytes per element, numpy dtype to view the bytes, torch dtype of the result)
    "F32": (4, np.float32, torch.float32),
    "F16": (2, np.float16, torch.float16),
    "BF16": (2, np.uint16, torch.bfloat16),
    "F64": (8, np.float64, torch.float64),
    "I64": (8, np.int64, torch.int32),
    "I32": (4, np.int32, torch.int32),
    "I16": (2, np.int16, torch.int32),
    "I8": (1, np.int8, torch.int32),
    "U8": (1, np.uint8, torch.int32),
    "BOOL": (1, np.uint8, torch.int32),
}
_WRITE_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                torch.float64: "F64", torch.int64: "I64", torch.int32: "I32"}


class TensorInfo:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, shape, begin, end, file


class SafetensorsFile:
    """One .safetensors file, memory-mapped."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"could not open {path} ({e.strerror})") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors header length")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        def no_duplicates(pairs):
            # two entries of one name: the reference stops (qwen_infer.c:345-350); Python's parser would keep the last
            seen = {}
            for k, v in pairs:
                if k in seen:
                    raise SafetensorsError(f"{path}: duplicate tensor name in the header: {k}")
                seen[k] = v
            return seen

        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"), object_pairs_hook=no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        self.tensors: Dict[str, TensorInfo] = {}
        for name, e in header.items():
            if not isinstance(e, dict) or "dtype" not in e or "shape" not in e or "data_offsets" not in e:
                raise SafetensorsError(f"{path}: tensor '{name}' lacks dtype, shape or data_offsets")
            dtype, shape, off = e["dtype"], e["shape"], e["data_offsets"]
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype '{dtype}'")
            if not isinstance(shape, list) or len(shape) > 8 or not all(isinstance(s, int) and s >= 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor '{name}' has a bad shape {shape}")
            if (not isinstance(off, list) or len(off) != 2 or not all(isinstance(o, int) for o in off)
                    or not 0 <= off[0] <= off[1] <= data_len):
                raise SafetensorsError(f"{path}: tensor '{name}' has offsets {off} outside the data section ({data_len} bytes)")
            count = 1
            for s in shape:
                count *= s
            if count * _DTYPES[dtype][0] != off[1] - off[0]:
                raise SafetensorsError(f"{path}: tensor '{name}' of shape {shape} and dtype {dtype} "
                                       f"does not fill its {off[1] - off[0]} bytes")
            self.tensors[name] = TensorInfo(name, dtype, tuple(shape), off[0], off[1], self)

    def read(self, info: TensorInfo) -> torch.Tensor:
        _, np_dtype, t_dtype = _DTYPES[info.dtype]
        count = 1
        for s in info.shape:
            count *= s
        arr = np.frombuffer(self._mm, dtype=np_dtype, count=count, offset=self.data_start + info.begin)
        if info.dtype == "BF16":
            t = torch.from_numpy(arr.copy()).view(torch.bfloat16)
        elif t_dtype == torch.int32:
            wide = arr.astype(np.int64)
            if count and (wide.min() < -2**31 or wide.max() >= 2**31):
                raise SafetensorsError(f"{self.path}: integer tensor '{info.name}' does not fit in int32")
            t = torch.from_numpy(wide.astype(np.int32))
        else:
            t = torch.from_numpy(arr.copy())
        return t.reshape(info.shape)

    def close(self):
        try:
            self._mm.close()
        finally:
            self._f.close()


class Checkpoint:
    """All tensors of a model folder (or of one file), by name."""

    def __init__(self, path: str):
        self.files: List[SafetensorsFile] = []
        self.tensors: Dict[str, TensorInfo] = {}
        if os.path.isdir(path):
            single = os.path.join(path, "model.safetensors")
            index = os.path.join(path, "model.safetensors.index.json")
            if os.path.exists(single):
                self._add_file(single)
            elif os.path.exists(index):
                self._add_index(index)
            else:
                raise SafetensorsError(f"{path}: neither model.safetensors nor model.safetensors.index.json found")
        elif path.endswith(".index.json"):
            self._add_index(path)
        else:
            self._add_file(path)

    def _add_file(self, path: str, only: Optional[Iterable[str]] = None):
        f = SafetensorsFile(path)
        self.files.append(f)
        wanted = set(only) if only is not None else None
        for name, info in f.tensors.items():
            if wanted is not None and name not in wanted:
                continue
            if name in self.tensors:
                raise SafetensorsError(f"tensor '{name}' appears twice ({self.tensors[name].file.path} and {path})")
            self.tensors[name] = info
        if wanted is not None:
            lost = sorted(wanted - set(f.tensors))
            if lost:
                raise SafetensorsError(f"{path}: the index lists {len(lost)} tensors that this shard lacks, first '{lost[0]}'")

    def _add_index(self, path: str):
        try:
            with open(path, "r", encoding="utf-8") as fh:
                index = json.load(fh)
        except (OSError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"could not read {path}: {e}") from e
        wm = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(wm, dict) or not wm:
            raise SafetensorsError(f"{path}: no 'weight_map' object")
        shards: Dict[str, List[str]] = {}
        for name, shard in wm.items():
            if not isinstance(shard, str) or "/" in shard or "\\" in shard or ".." in shard or not shard:
                raise SafetensorsError(f"{path}: shard name {shard!r} is not a plain file name")
            shards.setdefault(shard, []).append(name)
        base = os.path.dirname(path)
        for shard in sorted(shards):
            self._add_file(os.path.join(base, shard), only=shards[shard])

    def names(self) -> List[str]:
        return list(self.tensors)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.tensors[name].shape

    def dtype(self, name: str) -> str:
        return self.tensors[name].dtype

    def tensor(self, name: str) -> torch.Tensor:
        info = self.tensors[name]
        return info.file.read(info)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Write CPU tensors in name order, each aligned to 8 bytes through header padding."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _WRITE_NAMES:
            raise SafetensorsError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _WRITE_NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
