"""Python face of the runner: torch tensors in, C ABI underneath.

Mirrors ``slopfab::cuda::LinearRunner`` (include/slopfab/cuda/linear.cuh:182-242 of the
reference): ``forward``, ``prepare`` + ``forward_prepared``, ``set_native``. The arena is
a caller-visible torch uint8 tensor, grown to the high-water mark like the reference's
``Workspace``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import COMPUTE_BF16, QuantWeight, check, lib, ptr


def stream_ptr(stream: torch.cuda.Stream | None = None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class LinearRunner:
    def __init__(self, stream: torch.cuda.Stream | None = None, device: str | torch.device = "cuda"):
        self.device = torch.device(device)
        self.stream = stream
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.sfq_runner_create(stream_ptr(stream), C.byref(handle)))
        self._h = handle
        self._ws = torch.empty(0, dtype=torch.uint8, device=self.device)
        self._activation = 0

    def close(self) -> None:
        if self._h:
            lib.sfq_runner_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def set_native(self, enable: bool) -> None:
        check(lib.sfq_runner_set_native(self._h, int(enable)))

    def native(self) -> bool:
        return bool(lib.sfq_runner_native(self._h))

    def set_activation(self, activation: int) -> None:
        """ACT_NONE, ACT_GELU_TANH, or ACT_SWIGLU (weight rows [gate | up]; the output then has out_features / 2 columns)."""
        check(lib.sfq_runner_set_activation(self._h, activation))
        self._activation = activation

    @staticmethod
    def workspace_bytes(w: QuantWeight, rows: int) -> int:
        n = C.c_size_t(0)
        check(lib.sfq_linear_workspace_bytes(C.byref(w), rows, COMPUTE_BF16, C.byref(n)))
        return n.value

    def reserve(self, nbytes: int) -> None:
        if self._ws.numel() < nbytes:
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)

    def forward(self, w: QuantWeight, x: torch.Tensor, y: torch.Tensor | None = None) -> torch.Tensor:
        rows = x.shape[0]
        if y is None:
            cols = w.out_features // 2 if self._activation == 2 else w.out_features
            y = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device)
        self.reserve(self.workspace_bytes(w, rows))
        check(lib.sfq_linear_forward(self._h, C.byref(w), ptr(x), rows, ptr(y), ptr(self._ws), self._ws.numel()))
        return y

    def forward_f32(self, w: QuantWeight, x: torch.Tensor) -> torch.Tensor:
        """fp32 activations in, fp32 out (the arm the DiT uses for its adaLN tables)."""
        rows = x.shape[0]
        y = torch.empty((rows, w.out_features), dtype=torch.float32, device=x.device)
        n = C.c_size_t(0)
        check(lib.sfq_linear_workspace_bytes(C.byref(w), rows, 1, C.byref(n)))
        self.reserve(n.value)
        check(lib.sfq_linear_forward_f32(self._h, C.byref(w), ptr(x), rows, ptr(y), ptr(self._ws), self._ws.numel()))
        return y

    def prepare(self, w: QuantWeight, rows_per_chunk: int):
        """Returns (prepared pointer or None, bytes consumed at the front of the arena)."""
        self.reserve(self.workspace_bytes(w, rows_per_chunk))
        prepared = C.c_void_p()
        used = C.c_size_t(0)
        check(lib.sfq_linear_prepare(self._h, C.byref(w), ptr(self._ws), self._ws.numel(), C.byref(prepared),
                                     C.byref(used)))
        return prepared.value, used.value

    def forward_prepared(self, w: QuantWeight, prepared, used: int, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
        check(lib.sfq_linear_forward_prepared(self._h, C.byref(w), prepared, ptr(x), rows, ptr(y),
                                              ptr(self._ws) + used, self._ws.numel() - used))
        return y
