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
(`RandomSource`: N(0, std) per tensor from (seed, tensor name); norm weights 1).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Callable

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


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


class RandomSource(WeightSource):
    """Seeded random weights for the tensors a model needs: every weight N(0, std), norm weights 1.0.

    Values depend on (seed, tensor name) and on the device they are drawn on; the
    model-folder writer always draws on the CPU, so a folder is reproducible.
    """

    def __init__(self, needs: dict[str, TensorNeed], seed: int, std: float = 0.02, device="cpu",
                 dtype: torch.dtype = torch.bfloat16):
        self.needs = {n: t for n, t in needs.items() if not t.optional}
        self.seed, self.std, self.device, self.dtype = int(seed), float(std), torch.device(device), dtype

    def shapes(self):
        return {n: tuple(t.shape) for n, t in self.needs.items()}

    def read(self, name):
        need = self.needs[name]
        if need.init == "ones":
            return torch.ones(need.shape, dtype=torch.float32, device=self.device)
        g = torch.Generator(device=self.device)
        g.manual_seed(_tensor_seed(self.seed, name))
        t = torch.empty(need.shape, dtype=torch.float32 if self.device.type == "cpu" else self.dtype,
                        device=self.device)
        t.normal_(0.0, self.std, generator=g)
        return t.to(self.dtype)

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
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Random-weights mode: write `config.json` and `model.safetensors` for a configuration and a seed."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    src = RandomSource(needs, seed, std, device="cpu", dtype=dtype)
    tensors = {}
    for name in src.shapes():
        t = src.read(name)
        tensors[name] = t if needs[name].init == "ones" and dtype == torch.float32 else t.to(dtype)
    (folder / "config.json").write_text(json.dumps(config_json, indent=2))
    st.write_safetensors(folder / "model.safetensors", tensors,
                         metadata={"format": "pt", "seed": seed, "std": std})
    return folder
