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
        self.use_partials = True  # few-token contractions may leave their K slices unadded for the next reader

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

    def stream(self, x) -> "ResidualStream":
        """`x` as a residual stream: itself if it is one already, else a 32-bit tensor wrapped."""
        return x if isinstance(x, ResidualStream) else ResidualStream(self, x)

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


class ResidualStream:
    """The 32-bit residual stream of a step, `[rows, width]`, as blocks and parts get it.

    Over few tokens (up to a few hundred: the kernel library says how many) a contraction into the stream is cut
    along K over the SMs and leaves its slices unadded (`add_linear`); whoever reads the stream next adds them. That hand-over is this object's business, not the
    parts': `data` adds pending slices before it returns the tensor, so a part written against `data` (read it,
    update it in place) is always right. A reader that can add the slices while it reads, in the same pass over
    memory (the RMSNorm kernel), asks for `take()` instead and gets the tensor and the slices."""

    def __init__(self, runtime: Runtime, tensor: torch.Tensor):
        if tensor.dtype != torch.float32:
            raise ValueError("the residual stream is 32-bit in every mode")
        self.rt = runtime
        self._tensor = tensor
        self._pending = None

    @property
    def shape(self):
        return self._tensor.shape

    @property
    def data(self) -> torch.Tensor:
        """The stream's tensor with everything added; it may be read and updated in place."""
        if self._pending is not None:
            ps, self._pending = self._pending, None
            ops.add_partials(self._tensor, ps)
        return self._tensor

    def take(self):
        """(tensor, pending slices or None) for a reader that adds the slices itself, in the stream too: after
        the reader's kernel the tensor must hold the sum."""
        ps, self._pending = self._pending, None
        return self._tensor, ps

    def add_linear(self, a, w, bias=None) -> None:
        """stream += a @ w.T (+ bias). Over few tokens the slices may stay pending until the next reader."""
        rt = self.rt
        if rt.use_partials and bias is None and ops.gemm_partial_supported(a, w):
            x = self.data  # slices of an earlier contraction go in first
            self._pending = ops.gemm_partial(a, w, rt.err)
            assert x is self._tensor
        else:
            ops.gemm(a, w, self.data, ops.EPI_RESIDUAL, bias, rt.err)

    def add(self, delta: torch.Tensor) -> None:
        """stream += delta (any float dtype, same shape)."""
        self.data.add_(delta)

    def drop_pending(self) -> None:
        """Forget unadded slices: the stream will not be read again (no logits are wanted)."""
        self._pending = None
