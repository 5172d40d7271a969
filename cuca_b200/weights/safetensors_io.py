"""Reading and writing safetensors files without any helper library.

Format (src/provider/local/convert/safetensors.rs:1-24 of the reference): an
8-byte little-endian header length, a JSON header `{name: {dtype, shape,
data_offsets}}`, then the raw little-endian data. A folder is read through
`model.safetensors.index.json` (`weight_map`) when present, else
`model.safetensors`, else every `*.safetensors`
(src/provider/local/convert/hf.rs:26-28,97-110).
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype -> (numpy dtype used to read the bytes, torch dtype of the result)
_DTYPES = {
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),
    "F64": (np.float64, torch.float64),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32",
          torch.int64: "I64", torch.float64: "F64"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    file: Path
    begin: int  # absolute byte offsets in `file`
    end: int


def read_header(path: Path) -> dict[str, TensorInfo]:
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file")
        try:
            header = json.loads(f.read(n))
        except ValueError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from e
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dtype = meta["dtype"]
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor `{name}` has dtype {dtype}, which this engine does not read")
        lo, hi = meta["data_offsets"]
        shape = tuple(int(s) for s in meta["shape"])
        want = int(np.prod(shape, dtype=np.int64)) * np.dtype(_DTYPES[dtype][0]).itemsize if shape else \
            np.dtype(_DTYPES[dtype][0]).itemsize
        if hi - lo != want or base + hi > size:
            raise SafetensorsError(f"{path}: tensor `{name}` {dtype}{list(shape)} does not match its {hi - lo} bytes")
        out[name] = TensorInfo(name, dtype, shape, path, base + lo, base + hi)
    return out


def folder_index(model_dir) -> dict[str, TensorInfo]:
    """Every tensor of a model folder by name; a name in two files is an error."""
    model_dir = Path(model_dir)
    idx = model_dir / "model.safetensors.index.json"
    if idx.is_file():
        files = sorted({model_dir / f for f in json.loads(idx.read_text())["weight_map"].values()})
    elif (model_dir / "model.safetensors").is_file():
        files = [model_dir / "model.safetensors"]
    else:
        files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise SafetensorsError(f"{model_dir}: no safetensors file in the model folder")
    out: dict[str, TensorInfo] = {}
    for f in files:
        for name, info in read_header(f).items():
            if name in out:
                raise SafetensorsError(f"tensor `{name}` is in both {out[name].file.name} and {f.name}")
            out[name] = info
    return out


def read_tensor(info: TensorInfo) -> torch.Tensor:
    """The tensor as stored (bf16 stays bf16, 32-bit stays 32-bit); integer tables come back as int32."""
    np_dtype, torch_dtype = _DTYPES[info.dtype]
    count = (info.end - info.begin) // np.dtype(np_dtype).itemsize
    arr = np.fromfile(info.file, dtype=np_dtype, count=count, offset=info.begin).reshape(info.shape)
    t = torch.from_numpy(arr)
    if info.dtype == "BF16":
        t = t.view(torch.bfloat16)
    if not t.dtype.is_floating_point and t.dtype != torch.bool:
        t = t.to(torch.int32)
    return t


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor `{name}`: dtype {t.dtype} cannot be written")
        raw = t.view(torch.uint16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * ((8 - len(head) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
