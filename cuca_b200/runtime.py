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
    4: "a kernel found its shared memory laid out otherwise than its budget assumes",
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
        # residual streams whose last contraction left its K slices unadded (decode): stream address -> PartialSums
        self.pending: dict = {}
        self.use_partials = True

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

    # ---------------------------------------------------------------- partial sums on the residual stream
    def linear_into_stream(self, a, w, stream, bias=None) -> None:
        """stream += a @ w.T. Over few tokens the contraction is cut along K over the SMs and leaves its slices
        unadded; the next reader of the stream (a norm) adds them while it reads, which spares the contraction a
        second pass through memory at its end. `take_pending` / `flush` hand the slices over."""
        if self.use_partials and bias is None and ops.gemm_partial_supported(a, w):
            if stream.data_ptr() in self.pending:
                self.flush(stream)
            self.pending[stream.data_ptr()] = ops.gemm_partial(a, w, self.err)
        else:
            ops.gemm(a, w, stream, ops.EPI_RESIDUAL, bias, self.err)

    def take_pending(self, stream):
        return self.pending.pop(stream.data_ptr(), None)

    def flush(self, stream) -> None:
        """Add pending slices into the stream now (for a reader that does not add them itself)."""
        ps = self.pending.pop(stream.data_ptr(), None)
        if ps is not None:
            ops.add_partials(stream, ps)

    def check_device_errors(self) -> None:
        """Read the error word (synchronises); raise if a kernel recorded a fault."""
        code = int(self.err.item())
        if code:
            self.raise_device_error(code)

    def raise_device_error(self, code: int) -> None:
        """A kernel recorded `code` (read by the caller, e.g. along with a step's sampled tokens): clear the
        word and raise."""
        self.err.zero_()
        raise DeviceFault(_ERR_TEXT.get(code, f"device error {code}"))
