"""Binding checkpoint tensors to parts by name.

The parts of a model say which tensors they expect (`TensorNeed` by name); the
loader compares that list with what a source offers and raises ONE
`WeightsError` that lists every missing tensor, every unexpected tensor and
every wrong shape (the reference reports these per tensor:
src/provider/local/model/layout.rs:166-175, model/cpu.rs:762-767,
convert/tensors.rs:899-904). A tensor is read as stored (bfloat16 stays
bfloat16, 32-bit stays 32-bit, integer tables become int32); binding then casts
matrices to the compute dtype and leaves vectors marked `keep_fp32` in 32-bit.

Sources: a model folder (`FolderSource`) or seeded random weights
(`RandomSource`: N(0, std) per element from (seed, tensor name, element number); norm weights 1
or 1 + N(0, norm_std)).
"""
from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path
from typing import Callable

import numpy as np
import torch

from ..parts.base import TensorNeed
from . import safetensors_io as st

# wrapper prefixes the reference strips (src/provider/local/convert/tensors.rs:643-654)
_WRAPPER_PREFIXES = ("model.language_model.", "language_model.model.")


class WeightsError(ValueError):
    """Missing / unexpected tensors or wrong shapes; `.missing`, `.unexpected`, `.wrong_shape` hold them."""

    def __init__(self, missing, unexpected, wrong_shape, where: str = ""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"the weights{' in ' + where if where else ''} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


class WeightSource:
    def shapes(self) -> dict[str, tuple]:  # pragma: no cover - interface
        raise NotImplementedError

    def read(self, name: str) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def describe(self) -> str:
        return ""


class FolderSource(WeightSource):
    """`config.json` + safetensors in a folder."""

    def __init__(self, model_dir):
        self.dir = Path(model_dir)
        raw = st.folder_index(self.dir)
        self._index = {}
        for name, info in raw.items():
            short = name
            for p in _WRAPPER_PREFIXES:
                if name.startswith(p):
                    short = "model." + name[len(p):]
            if short in self._index:
                raise st.SafetensorsError(f"tensors `{name}` and `{self._index[short].name}` both bind to `{short}`")
            self._index[short] = info

    def shapes(self):
        return {n: i.shape for n, i in self._index.items()}

    def read(self, name):
        return st.read_tensor(self._index[name])

    def describe(self):
        return str(self.dir)


def tensor_key(seed: int, name: str) -> int:
    """64-bit key of one tensor's random stream, from (seed, tensor name)."""
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_SUM_SIGMA = math.sqrt(65536.0 ** 2 - 1.0)  # deviation of the sum of twelve uniform 16-bit fields


def normal_scale(std: float) -> np.float32:
    return np.float32(std / (2.0 * _SUM_SIGMA))


def host_normal(key: int, first: int, n: int, mean: float, std: float) -> np.ndarray:
    """Elements first..first+n-1 of the tensor with this key as float32: element i is a function of (key, i)
    alone. Outputs 3i, 3i+1, 3i+2 of a SplitMix64 stream that starts at `key` give twelve 16-bit fields whose sum
    is near-normal; v = (2 sum - 12 * 65535) * scale, then mean + v, each one 32-bit rounding. The device kernel
    (`cuca_random_normal`) does the same arithmetic, so host-drawn and device-drawn weights are the same bits."""
    out = np.empty(n, dtype=np.float32)
    scale, mean32 = normal_scale(std), np.float32(mean)
    chunk = 1 << 16  # temporaries stay in cache
    with np.errstate(over="ignore"):
        for lo in range(0, n, chunk):
            m = min(chunk, n - lo)
            e = np.arange(first + lo, first + lo + m, dtype=np.uint64)
            total = np.zeros(m, dtype=np.int64)
            for j in range(3):
                z = np.uint64(key) + (np.uint64(3) * e + np.uint64(j + 1)) * _GOLDEN
                z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
                z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
                z = z ^ (z >> np.uint64(31))
                for shift in (0, 16, 32, 48):
                    total += ((z >> np.uint64(shift)) & np.uint64(0xFFFF)).astype(np.int64)
            v = (2 * total - 12 * 65535).astype(np.float32) * scale
            out[lo:lo + m] = mean32 + v
    return out


class RandomSource(WeightSource):
    """Seeded random weights for the tensors a model needs: every weight N(0, std); norm weights
    (`init="ones"`) 1.0, or 1 + N(0, norm_std) when `norm_std` is given so that a swapped or dropped norm
    weight changes the logits. Optional tensors that the model lists (biases that its configuration
    switches on) are drawn too. A value depends on (seed, tensor name, element number) only: drawn on the host
    or by the device kernel, whole or in pieces, the bits are the same."""

    def __init__(self, needs: dict[str, TensorNeed], seed: int, std: float = 0.02, device="cpu",
                 dtype: torch.dtype = torch.bfloat16, norm_std: float = 0.0):
        self.needs = dict(needs)
        self.seed, self.std, self.device, self.dtype = int(seed), float(std), torch.device(device), dtype
        self.norm_std = float(norm_std)

    def shapes(self):
        return {n: tuple(t.shape) for n, t in self.needs.items()}

    def read(self, name):
        need = self.needs[name]
        ones = need.init == "ones"
        if ones and self.norm_std == 0.0:
            return torch.ones(need.shape, dtype=torch.float32, device=self.device)
        mean, std = (1.0, self.norm_std) if ones else (0.0, self.std)
        dtype = self.dtype  # what a folder of this dtype would hold (binding widens norm weights to 32-bit)
        n = 1
        for s in need.shape:
            n *= int(s)
        key = tensor_key(self.seed, name)
        if self.device.type == "cuda":
            from ..kernels import ops
            t = torch.empty(need.shape, dtype=dtype, device=self.device)
            ops.random_normal(t, key, 0, mean, float(normal_scale(std)))
            return t
        return torch.from_numpy(host_normal(key, 0, n, mean, std)).view(need.shape).to(dtype)

    def describe(self):
        return f"random weights (seed {self.seed}, std {self.std})"


def check_tensors(needs: dict[str, TensorNeed], shapes: dict[str, tuple],
                  ignorable: Callable[[str], bool] = lambda n: False, where: str = "") -> None:
    missing = [n for n, t in needs.items() if not t.optional and n not in shapes]
    unexpected = [n for n in shapes if n not in needs and not ignorable(n)]
    wrong = [(n, tuple(needs[n].shape), tuple(shapes[n])) for n in shapes
             if n in needs and tuple(needs[n].shape) != tuple(shapes[n])]
    if missing or unexpected or wrong:
        raise WeightsError(sorted(missing), sorted(unexpected), sorted(wrong), where)


def binder(needs: dict[str, TensorNeed], source: WeightSource, device, compute_dtype: torch.dtype):
    """`get(name)`: the tensor on `device`, or None for an absent optional one."""
    shapes = source.shapes()

    def get(name: str):
        need = needs[name]
        if name not in shapes:
            if need.optional:
                return None
            raise WeightsError([name], [], [], source.describe())
        t = source.read(name)
        if t.dtype.is_floating_point:
            t = t.to(device=device, dtype=torch.float32 if need.keep_fp32 else compute_dtype)
        else:
            t = t.to(device=device, dtype=torch.int32)
        return t.contiguous()

    return get


def write_model_folder(folder, config_json: dict, needs: dict[str, TensorNeed], seed: int, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16, norm_std: float = 0.0, device="cpu") -> Path:
    """Random-weights mode: write `config.json` and `model.safetensors` for a configuration and a seed.
    `device`: where the values are drawn (the bits are the same; a CUDA device draws a large model in seconds)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    src = RandomSource(needs, seed, std, device=device, dtype=dtype, norm_std=norm_std)
    tensors = {}
    for name in src.shapes():
        t = src.read(name).cpu()
        tensors[name] = t if needs[name].init == "ones" and dtype == torch.float32 else t.to(dtype)
    (folder / "config.json").write_text(json.dumps(config_json, indent=2))
    st.write_safetensors(folder / "model.safetensors", tensors,
                         metadata={"format": "pt", "seed": seed, "std": std, "norm_std": norm_std})
    return folder
