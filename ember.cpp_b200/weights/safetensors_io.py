"""Reading and writing the safetensors container.

The format as ember.cpp reads it: an 8-byte little-endian header length, a JSON header, then the
data block (safetensors_loader.cpp:151-164); per tensor `dtype`, `shape` and `data_offsets`
[begin, end) into the data block (:459-475); `__metadata__` is skipped (:454); reads are range
checked against the file (:261-281).  A folder may hold one `model.safetensors` or shards named
by `model.safetensors.index.json`'s `weight_map` (:321-409).

Tensors keep the type they are stored in: BF16 stays bfloat16, F32 stays float32; F16 becomes
float32 (exact); integer tables become int32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
           "I32": (torch.int32, 4), "I64": (torch.int64, 8)}
_NAMES = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16", torch.int32: "I32", torch.int64: "I64"}


class SafetensorsError(ValueError):
    pass


class UnreadTensor:
    """A tensor of the file whose stored type this library does not read (BOOL, U8, F64, ...): its
    name, shape and type are known, its values are not fetched.  Checkpoints carry such tensors as
    buffers that no model wants (GPT-2's causal mask is saved as BOOL or U8 by some writers); the
    loader complains only if a model asks for one."""

    def __init__(self, dtype_name: str, shape):
        self.dtype_name, self.shape = dtype_name, tuple(shape)


def read_header(path: str) -> tuple[dict, int]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: shorter than its 8-byte header length")
        (n,) = struct.unpack("<Q", head)
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file ({size} bytes)")
        raw = f.read(n)
    try:
        header = json.loads(raw)
    except json.JSONDecodeError as e:
        raise SafetensorsError(f"{path}: header is not JSON ({e}); it starts {raw[:40]!r}") from None
    return header, 8 + n


def read_file(path: str) -> dict[str, torch.Tensor]:
    """All tensors of one file, as views of a private memory map (copy-on-write, so that torch may
    treat them as writable without touching the file)."""
    header, base = read_header(path)
    size = os.path.getsize(path)
    out: dict[str, torch.Tensor] = {}
    if size == base:
        return out
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt = str(meta.get("dtype", "")).upper()
        shape = [int(s) for s in meta["shape"]]
        if dt not in _DTYPES:
            out[name] = UnreadTensor(str(meta.get("dtype")), shape)
            continue
        tdt, width = _DTYPES[dt]
        begin, end = (int(v) for v in meta["data_offsets"])
        numel = 1
        for s in shape:
            numel *= s
        if end - begin != numel * width:
            raise SafetensorsError(f"{path}: tensor {name!r} of shape {shape} and dtype {dt} needs {numel * width} "
                                   f"bytes, its offsets give {end - begin}")
        if begin < 0 or base + end > size:
            raise SafetensorsError(f"{path}: tensor {name!r} lies at bytes [{begin}, {end}) of a data block of "
                                   f"{size - base} bytes")
        if numel == 0:
            t = torch.empty(shape, dtype=tdt)
        else:
            t = torch.frombuffer(mm, dtype=tdt, count=numel, offset=base + begin).reshape(shape)
        if tdt == torch.float16:
            t = t.to(torch.float32)
        elif tdt == torch.int64:
            t = t.to(torch.int32)
        out[name] = t
    return out


def read_folder(folder: str) -> dict[str, torch.Tensor]:
    """`model.safetensors`, or the shards that `model.safetensors.index.json` names."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(single):
        return read_file(single)
    if os.path.isfile(index):
        with open(index) as f:
            weight_map = json.load(f).get("weight_map", {})
        out: dict[str, torch.Tensor] = {}
        for shard in sorted(set(weight_map.values())):
            out.update(read_file(os.path.join(folder, shard)))
        return out
    raise SafetensorsError(f"{folder}: no model.safetensors (or model.safetensors.index.json) in the model folder")


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous().reshape(-1)
            if t.numel():
                f.write(t.view(torch.uint8).numpy().data)
