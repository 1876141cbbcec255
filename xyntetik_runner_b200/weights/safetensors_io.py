"""Reading and writing the safetensors container, by tensor name.

The file is: an 8-byte little-endian header length, a JSON header that maps
each name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the bytes.  The reference reads its
own container (GGUF) the same way -- a directory of named, typed, shaped
tensors over one memory map, with offsets checked against the file size
(src/gguf.h:62-71, src/model.c:121-170) -- and that discipline is kept here:
every offset is checked before a view is made.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Optional, Dict, Iterable, Iterator, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
HEADER_MAX = 100 << 20


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int          # absolute byte offset in the file
    nbytes: int


class SafetensorsFile:
    """One mapped file; tensors are views of the map until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen < 2 or hlen > HEADER_MAX or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + hlen
        self.tensors: Dict[str, TensorInfo] = {}
        for name, ent in header.items():
            try:
                dt, shape, (b, e) = ent["dtype"], tuple(int(s) for s in ent["shape"]), ent["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            tdt, esz = _DTYPES[dt]
            n = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor '{name}' has a negative extent")
                n *= s
            if b < 0 or e < b or e - b != n * esz or base + e > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' data_offsets [{b}, {e}) do not match shape {list(shape)} "
                    f"of {dt} or lie outside the file")
            self.tensors[name] = TensorInfo(name, tdt, shape, base + b, e - b)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.tensors)

    def get(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the mapped bytes (copy before writing)."""
        info = self.tensors[name]
        if info.nbytes == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # the map is read-only; views are never written
            flat = torch.frombuffer(self._map, dtype=torch.uint8, count=info.nbytes, offset=info.begin)
        return flat.view(info.dtype).reshape(info.shape)

    def close(self) -> None:
        # views may still reference the map; let the garbage collector take it
        self._f.close()


def read_weight_map(model_dir: str) -> Optional[Dict[str, str]]:
    """{tensor name: shard file} of model.safetensors.index.json, or None for a folder with a single file."""
    if os.path.isfile(os.path.join(model_dir, "model.safetensors")):
        return None
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if not os.path.isfile(index):
        raise SafetensorsError(f"{model_dir}: no model.safetensors (nor an index) found")
    try:
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map")
    except (OSError, ValueError) as e:
        raise SafetensorsError(f"{index}: {e}") from None
    if not isinstance(wm, dict) or not wm or not all(isinstance(k, str) and isinstance(v, str) for k, v in wm.items()):
        raise SafetensorsError(f"{index}: weight_map must map tensor names to file names")
    for fn in wm.values():
        if os.path.basename(fn) != fn:
            raise SafetensorsError(f"{index}: shard '{fn}' is not a plain file name")
    return wm


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The safetensors files of a model folder: the single file, or the shards an index names."""
    wm = read_weight_map(model_dir)
    if wm is None:
        return [SafetensorsFile(os.path.join(model_dir, "model.safetensors"))]
    out = []
    for fn in sorted(set(wm.values())):
        path = os.path.join(model_dir, fn)
        if not os.path.isfile(path):
            raise SafetensorsError(f"{model_dir}: the index names shard '{fn}', which is not there")
        out.append(SafetensorsFile(path))
    return out


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None,
                      layout: List[Tuple[str, torch.dtype, Tuple[int, ...]]] = None) -> None:
    """Write tensors to `path`.

    With `layout` (name, dtype, shape for every tensor, in order) the header is
    written first and `tensors` is consumed as a stream, so a model larger than
    host memory can be written one tensor at a time.  Without it the tensors
    are collected first.
    """
    if layout is None:
        tensors = list(tensors)
        layout = [(n, t.dtype, tuple(t.shape)) for n, t in tensors]
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, dt, shape in layout:
        if dt not in _NAMES:
            raise SafetensorsError(f"cannot write dtype {dt}")
        n = 1
        for s in shape:
            n *= s
        nb = n * _DTYPES[_NAMES[dt]][1]
        header[name] = {"dtype": _NAMES[dt], "shape": list(shape), "data_offsets": [off, off + nb]}
        off += nb
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        it: Iterator[Tuple[str, torch.Tensor]] = iter(tensors)
        for name, dt, shape in layout:
            n2, t = next(it)
            if n2 != name or t.dtype != dt or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor stream does not follow the layout at '{name}'")
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
