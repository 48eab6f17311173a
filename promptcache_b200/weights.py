"""Reader of safetensors checkpoints: an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets), then the raw little-endian data.  Tensors are read through one memory map of the
file and copied to the target device one by one; nothing else of the file format is needed, so no package is imported."""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Iterator, Optional, Tuple

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64, "I64": torch.int64,
           "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


def read_header(path: str) -> Tuple[Dict[str, dict], int]:
    """(name -> {dtype, shape, data_offsets}, offset of the data section)."""
    with open(path, "rb") as fh:
        raw = fh.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: not a safetensors file (no header length)")
        n = struct.unpack("<Q", raw)[0]
        if n <= 0 or n > (100 << 20):
            raise ValueError(f"{path}: implausible header length {n}")
        meta = json.loads(fh.read(n).decode("utf-8"))
    meta.pop("__metadata__", None)
    return meta, 8 + n


def iter_tensors(path: str, device="cpu", dtype: Optional[torch.dtype] = None) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, tensor on `device`).  Floating tensors are converted to `dtype` when one is given; integer tables keep
    their type."""
    meta, base = read_header(path)
    with open(path, "rb") as fh:
        mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name, info in meta.items():
                dt = _DTYPES.get(info["dtype"])
                if dt is None:
                    raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
                lo, hi = info["data_offsets"]
                shape = tuple(info["shape"])
                count = 1
                for s in shape:
                    count *= s
                if hi - lo != count * torch.empty((), dtype=dt).element_size():
                    raise ValueError(f"{path}: tensor {name}: {hi - lo} bytes do not fit shape {shape}")
                if count == 0:
                    t = torch.empty(shape, dtype=dt)
                else:
                    t = torch.frombuffer(bytearray(mm[base + lo:base + hi]), dtype=dt).reshape(shape)
                t = t.to(device)
                if dtype is not None and t.is_floating_point():
                    t = t.to(dtype)
                yield name, t
        finally:
            mm.close()


def load_file(path: str, device="cpu", dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    return dict(iter_tensors(path, device, dtype))


def save_file(tensors: Dict[str, torch.Tensor], path: str) -> None:
    """Write a checkpoint in the same format (tests and tools build small random models with it)."""
    names = {v: k for k, v in _DTYPES.items()}
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    js = json.dumps(header, separators=(",", ":")).encode("utf-8")
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(js)))
        fh.write(js)
        for raw in blobs:
            fh.write(raw)
