"""What every part needs of its surroundings: device, compute dtype, the error word, projections."""
from __future__ import annotations

import torch

from .kernels import library, ops


class DeviceFault(RuntimeError):
    """A kernel recorded a bad index (token id, page id) or a wait that ran out."""


_ERR_TEXT = {
    1: "a token id or position outside its table reached a kernel",
    2: "a page id outside the pool, or a position without a page, reached a kernel",
    3: "a bounded wait inside a kernel ran out",
}


class Runtime:
    """Device, compute dtype (float32: true 32-bit everywhere; bfloat16: serving precision) and shared helpers."""

    def __init__(self, device="cuda:0", dtype: torch.dtype = torch.bfloat16):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, not {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        if self.device.type != "cuda":
            raise library.KernelLibraryError(
                "cuca_b200 runs on a CUDA device only: there is no CPU path (device given: %s)" % device)
        if not torch.cuda.is_available():
            raise library.KernelLibraryError("no CUDA device is visible: cuca_b200 has no CPU path")
        library.load()
        torch.cuda.set_device(self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ---------------------------------------------------------------- helpers
    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def linear(self, a, w, out=None, epilogue=ops.EPI_STORE, bias=None, out_dtype=None):
        """out = epilogue(a @ w.T): store, add to the 32-bit stream, or SwiGLU over stacked [gate; up]."""
        n = w.shape[0] // 2 if epilogue == ops.EPI_SWIGLU else w.shape[0]
        if out is None:
            out = self.empty(a.shape[0], n, dtype=out_dtype or self.dtype)
        ops.gemm(a, w, out, epilogue, bias, self.err)
        return out

    def check_device_errors(self) -> None:
        """Read the error word (synchronises); raise if a kernel recorded a fault."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            raise DeviceFault(_ERR_TEXT.get(code, f"device error {code}"))
