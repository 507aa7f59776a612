"""Reading and writing .safetensors files: an 8-byte little-endian header length, a JSON header
(name -> dtype, shape, data_offsets) and the raw little-endian tensor data.

Tensors are memory-mapped and keep their stored element type; nothing is converted here.
(lite_llama converts a Hugging Face checkpoint into a ``.pth`` of its own names first,
lite_llama/executor/weight_convert.py:182-252, and reads that with ``torch.load(mmap=True)``,
lite_llama/executor/model_executor.py:92-117; here the checkpoint's own file is the input.)
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, List, Union

import torch

_TO_TORCH = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: Union[str, Path]):
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", raw)
        if hlen > 100 * 1024 * 1024:
            raise SafetensorsError(f"{path}: header length {hlen} is implausible")
        try:
            header = json.loads(f.read(hlen))
        except ValueError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    return header, 8 + hlen


def read_file(path: Union[str, Path]) -> Dict[str, torch.Tensor]:
    """name -> tensor backed by a read-only memory map of the file."""
    header, base = read_header(path)
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _TO_TORCH:
            raise SafetensorsError(f"{path}: tensor {name} has unsupported element type {meta['dtype']}")
        dtype = _TO_TORCH[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        numel = 1
        for s in meta["shape"]:
            numel *= s
        if hi - lo != numel * torch.empty((), dtype=dtype).element_size():
            raise SafetensorsError(f"{path}: tensor {name} has {hi - lo} bytes for shape {meta['shape']}")
        if numel == 0:
            out[name] = torch.empty(meta["shape"], dtype=dtype)
            continue
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; tensors are never written to
            t = torch.frombuffer(mm, dtype=dtype, count=numel, offset=base + lo)
        out[name] = t.reshape(meta["shape"])
    return out


def read_folder(folder: Union[str, Path]) -> Dict[str, torch.Tensor]:
    """All tensors of a model folder: model.safetensors, or the shards an index file lists."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    files: List[Path]
    if index.is_file():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        files = [folder / n for n in names]
    elif (folder / "model.safetensors").is_file():
        files = [folder / "model.safetensors"]
    else:
        files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {folder}")
    out: Dict[str, torch.Tensor] = {}
    for f in files:
        out.update(read_file(f))
    return out


def write_file(path: Union[str, Path], tensors: Dict[str, torch.Tensor]) -> None:
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _FROM_TORCH:
            raise SafetensorsError(f"tensor {name}: element type {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _FROM_TORCH[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(memoryview(t.view(torch.uint8).reshape(-1).numpy()))      # no copy of the tensor's bytes
