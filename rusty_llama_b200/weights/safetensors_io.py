"""Reading and writing safetensors files, with every malformed file an error.

Layout of a file: an 8-byte little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}` and the raw
little-endian tensor bytes.  The reference's counterpart is its GGUF reader,
whose bounds, overflow and alignment checks (src/model.rs:2013-2038) and
"truncated file is an Err, not a panic" rule (tests/integration.rs:107-120) are
kept; the container itself is this library's own choice.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch

from ..errors import WeightsError

# dtype name -> (bytes per element, numpy dtype used to view it, torch dtype)
_DTYPES = {
    "F32": (4, np.float32, torch.float32),
    "BF16": (2, np.uint16, torch.bfloat16),
    "F16": (2, np.float16, torch.float16),
    "I32": (4, np.int32, torch.int32),
    "I64": (8, np.int64, torch.int64),
}
_TORCH_TO_NAME = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32", torch.int64: "I64"}

_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """One mapped file; tensors are views of the mapping until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._fh = open(path, "rb")
        except OSError as e:
            raise WeightsError(f"cannot open '{path}': {e}") from None
        if size < 8:
            self._fh.close()
            raise WeightsError(f"'{path}' is {size} bytes, too short for a safetensors header")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            self.close()
            raise WeightsError(f"'{path}' is truncated or not safetensors: header of {hlen} bytes in a file of {size}")
        try:
            header = json.loads(self._map[8 : 8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            self.close()
            raise WeightsError(f"'{path}': header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            self.close()
            raise WeightsError(f"'{path}': header must be a JSON object")
        self._data0 = 8 + hlen
        data_size = size - self._data0
        self.metadata = header.pop("__metadata__", None) or {}
        self.tensors: Dict[str, TensorInfo] = {}
        spans: List[Tuple[int, int, str]] = []
        for name, meta in header.items():
            try:
                dtype = meta["dtype"]
                shape = tuple(int(s) for s in meta["shape"])
                begin, end = (int(o) for o in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                self.close()
                raise WeightsError(f"'{path}': tensor '{name}' has a malformed header entry") from None
            if dtype not in _DTYPES:
                self.close()
                raise WeightsError(f"'{path}': tensor '{name}' has unsupported dtype '{dtype}'")
            count = 1
            for s in shape:
                if s < 0:
                    self.close()
                    raise WeightsError(f"'{path}': tensor '{name}' has a negative size in shape {shape}")
                count *= s
            nbytes = count * _DTYPES[dtype][0]
            if begin < 0 or end < begin or end > data_size or end - begin != nbytes:
                self.close()
                raise WeightsError(
                    f"'{path}': tensor '{name}' ({dtype}{list(shape)}, {nbytes} bytes) has offsets "
                    f"[{begin}, {end}) in a data section of {data_size} bytes: file truncated or corrupt"
                )
            self.tensors[name] = TensorInfo(name, dtype, shape, begin, end)
            spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                self.close()
                raise WeightsError(f"'{path}': tensors '{n0}' and '{n1}' overlap")

    def close(self) -> None:
        try:
            self._map.close()
        except (AttributeError, BufferError, ValueError):
            pass
        try:
            self._fh.close()
        except AttributeError:
            pass

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its bytes (copied out of the mapping)."""
        info = self.tensors[name]
        _, np_dtype, torch_dtype = _DTYPES[info.dtype]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=info.end - info.begin, offset=self._data0 + info.begin)
        arr = raw.copy().view(np_dtype).reshape(info.shape)
        t = torch.from_numpy(arr)
        if info.dtype == "BF16":
            t = t.view(torch.bfloat16)
        del raw
        return t


class Checkpoint:
    """All tensors of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self._files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
                paths = [os.path.join(model_dir, p) for p in sorted(set(weight_map.values()))]
            except (OSError, KeyError, TypeError, json.JSONDecodeError, UnicodeDecodeError) as e:
                raise WeightsError(f"cannot read the shard index '{index}': {e}") from None
        else:
            raise WeightsError(f"'{model_dir}' has neither model.safetensors nor model.safetensors.index.json")
        try:
            for p in paths:
                f = SafetensorsFile(p)
                self._files.append(f)
                for name in f.names():
                    if name in self._where:
                        raise WeightsError(f"tensor '{name}' is in both '{self._where[name].path}' and '{p}'")
                    self._where[name] = f
        except WeightsError:
            self.close()
            raise

    def close(self) -> None:
        for f in self._files:
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def names(self):
        return self._where.keys()

    def info(self, name: str) -> TensorInfo:
        return self._where[name].tensors[name]

    def read(self, name: str) -> torch.Tensor:
        return self._where[name].read(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Write CPU tensors in the order given, each 8-byte aligned through header padding."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = []
    for name, t in tensors.items():
        if t.dtype not in _TORCH_TO_NAME:
            raise WeightsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        t = t.detach().cpu().contiguous()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append(t)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in order:
            if t.numel() == 0:
                continue
            flat = t.view(torch.uint8) if t.dim() else t.reshape(1).view(torch.uint8)
            f.write(flat.numpy().tobytes())
