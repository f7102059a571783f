"""Reading and writing the safetensors container, without the library of that name.

Format as the reference reads it (src/model.cpp:169-219): an 8-byte little-endian
header length, a JSON header ``{name: {"dtype", "shape", "data_offsets": [begin, end]}}``
(plus an optional ``__metadata__`` object), then the raw little-endian data, offsets
relative to the end of the header.  The reference rejects headers above 100 MB
(:173-175) and silently drops tensors of other dtypes (:276-279); here a bad header,
an unknown dtype, or offsets that disagree with shape x element size are errors
that name the tensor.  Tensors are memory-mapped, not copied, until they are used.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import numpy as np
import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """name -> CPU tensor viewing the memory-mapped file (read-only; clone or move before writing)."""
    path = Path(path)
    size = path.stat().st_size
    if size < 8:
        raise SafetensorsError(f"{path}: too short to hold a safetensors header")
    f = open(path, "rb")
    (hlen,) = struct.unpack("<Q", f.read(8))
    if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
        raise SafetensorsError(f"{path}: header length {hlen} is implausible for a file of {size} bytes")
    try:
        header = json.loads(f.read(hlen))
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise SafetensorsError(f"{path}: the header is not valid JSON ({e})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: the header is not a JSON object")
    base = 8 + hlen
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
    buf = np.frombuffer(mm, dtype=np.uint8)
    out: dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype_name, shape, (begin, end) = meta["dtype"], list(meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: tensor '{name}' has a malformed header entry") from None
        if dtype_name not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype_name} "
                                   f"(supported: {sorted(_DTYPES)})")
        tdtype, esize = _DTYPES[dtype_name]
        numel = 1
        for s in shape:
            numel *= int(s)
        if end - begin != numel * esize or begin < 0 or base + end > size:
            raise SafetensorsError(f"{path}: tensor '{name}' spans bytes [{begin}, {end}) but shape {shape} of "
                                   f"{dtype_name} needs {numel * esize} (file holds {size - base} data bytes)")
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the map is read-only on purpose; nothing writes through it
            raw = torch.from_numpy(buf[base + begin: base + end])
        out[name] = raw.view(tdtype).reshape(shape) if numel else torch.empty(shape, dtype=tdtype)
    return out


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Writes CPU tensors in name order; data offsets are 8-byte aligned by padding the header."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which this writer does not store")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
