"""Reading and writing the safetensors container, without a library.

Format (the one the reference parses in include/firefly/io/safetensors.h:50-99):
eight bytes of little-endian header length, a JSON header that maps each tensor
name to ``{dtype, shape, data_offsets}`` (offsets relative to the end of the
header; the ``__metadata__`` entry is skipped), then the raw little-endian data.
The file is memory-mapped; tensors are views into the mapping until they are
copied to the device.  Every offset is checked against the file size and
against shape x dtype, which the reference does not do.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int   # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file: header parsed and checked at open."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file too small to be safetensors ({size} bytes)")
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: invalid header size {hlen} for a file of {size} bytes")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dt_name, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if dt_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype '{dt_name}'")
            dtype, esize = _DTYPES[dt_name]
            shape = tuple(int(s) for s in shape)
            n = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension")
                n *= s
            if not (0 <= b <= e) or base + e > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' data_offsets [{b},{e}) lie outside the file")
            if e - b != n * esize:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' holds {e - b} bytes, shape {list(shape)} of {dt_name} "
                    f"needs {n * esize}")
            self.entries[name] = TensorEntry(name, dtype, shape, base + b, base + e)

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (read-only memory: copy before writing)."""
        try:
            ent = self.entries[name]
        except KeyError:
            raise SafetensorsError(f"{self.path}: tensor not found: {name}") from None
        n = 1
        for s in ent.shape:
            n *= s
        if n == 0:
            return torch.empty(ent.shape, dtype=ent.dtype)
        buf = memoryview(self._map)[ent.begin:ent.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=ent.dtype, count=n)
        return t.view(ent.shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through their memoryview
        try:
            self._map.close()
        except BufferError:
            pass
        self._fh.close()


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The weight files of a model folder: ``model.safetensors``, or the shards
    named by ``model.safetensors.index.json``."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as fh:
            wm = json.load(fh).get("weight_map", {})
        shards = sorted(set(wm.values()))
        if not shards:
            raise SafetensorsError(f"{index}: empty weight_map")
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in '{model_dir}'")


def save_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                     metadata: Mapping[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order: List[Tuple[str, torch.Tensor]] = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor '{name}')")
        t = t.detach().to("cpu").contiguous()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append((name, t))
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in order:
            if t.numel():
                fh.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                         t.reshape(1).view(torch.uint8).numpy().tobytes())
