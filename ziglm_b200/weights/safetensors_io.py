"""Reading and writing the safetensors container.

File layout (as the reference reads it, src/safetensors.zig:82-170): an 8-byte
little-endian header length, a JSON object mapping tensor names to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end
of the header), then the raw little-endian tensor bytes.  The reference maps
unknown dtypes to F32 silently (src/safetensors.zig:469-479) and keeps shapes in
reversed order; here unknown dtypes are an error and shapes stay as stored.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}

_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are zero-copy views of the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise SafetensorsError(f"{path} does not exist") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen < 2 or hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            if not isinstance(e, dict) or "dtype" not in e or "shape" not in e or "data_offsets" not in e:
                raise SafetensorsError(f"{path}: entry {name!r} lacks dtype, shape or data_offsets")
            dt = e["dtype"]
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            shape = tuple(int(s) for s in e["shape"])
            if any(s < 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has a negative extent {shape}")
            off = e["data_offsets"]
            if not (isinstance(off, list) and len(off) == 2):
                raise SafetensorsError(f"{path}: tensor {name!r} has malformed data_offsets {off!r}")
            begin, end = int(off[0]), int(off[1])
            count = 1
            for s in shape:
                count *= s
            if not (0 <= begin <= end <= data_len) or end - begin != count * _DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ({dt}{list(shape)}) has data_offsets [{begin}, {end}) that do not "
                    f"match its size or lie outside the {data_len} data bytes")
            self._entries[name] = (dt, shape, begin, end)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapped file (read-only; copy before writing)."""
        dt, shape, begin, end = self._entries[name]
        torch_dtype, _ = _DTYPES[dt]
        if end == begin:
            return torch.empty(shape, dtype=torch_dtype)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        # frombuffer warns about read-only memory; the loader only ever reads or copies.
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=torch_dtype)
        return t.reshape(shape)

    def close(self) -> None:
        # Views handed out keep the map alive through the buffer protocol.
        try:
            self._f.close()
        except Exception:
            pass


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write ``tensors`` (CPU or device) to ``path``; names are stored in the given order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order: List[Tuple[str, torch.Tensor]] = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append((name, t))
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((-len(raw)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for _, t in order:
            c = t.detach().to("cpu").contiguous()
            if c.numel():
                f.write(c.view(torch.uint8).numpy().tobytes() if c.dim() else
                        c.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(folder: str) -> Tuple[Dict[str, SafetensorsFile], Dict[str, str]]:
    """Open the weight file(s) of a model folder.

    Returns the open files by file name and a map from tensor name to file name.
    A single ``model.safetensors`` is what the reference reads
    (src/safetensors.zig:24-69); ``model.safetensors.index.json`` with shards is
    read as well.
    """
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    files: Dict[str, SafetensorsFile] = {}
    where: Dict[str, str] = {}
    if os.path.exists(single):
        f = SafetensorsFile(single)
        files["model.safetensors"] = f
        for n in f.names():
            where[n] = "model.safetensors"
        return files, where
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as fh:
            try:
                idx = json.load(fh)
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{index} is not valid JSON: {e}") from None
        wm = idx.get("weight_map") if isinstance(idx, dict) else None
        if not isinstance(wm, dict):
            raise SafetensorsError(f"{index}: no 'weight_map' object")
        for name, fname in wm.items():
            if fname not in files:
                files[fname] = SafetensorsFile(os.path.join(folder, fname))
            if name not in files[fname]:
                raise SafetensorsError(f"{index}: tensor {name!r} is not in {fname}")
            where[name] = fname
        return files, where
    raise SafetensorsError(f"{folder} holds neither model.safetensors nor model.safetensors.index.json")
