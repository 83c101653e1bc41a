"""ctypes face of the LoRA side branch (LoraRunner, include/slopfab/cuda/lora.cuh:14-37)."""
import ctypes as C

import numpy as np

from . import check, lib, ptr, stream_ptr


class LoraRunner:
    """y += (x A^T) B^T for the factor pairs attached under a key; keys are plain integers here."""

    def __init__(self):
        self._h = C.c_void_p()
        check(lib.sfq_lora_create(C.byref(self._h)))

    def close(self):
        if self._h:
            lib.sfq_lora_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def attach(self, key: int, a: np.ndarray, b: np.ndarray, row_offset: int = 0, out: int | None = None, staging=None):
        """a: fp32 [rank, in]; b: fp32 [out_total, rank]; rows [row_offset, row_offset + out) of b are used.
        staging = (host_ptr, device_ptr, offset) writes the bf16 bytes to host staging memory instead; returns the
        advanced offset."""
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        rank, k = a.shape
        out_total = b.shape[0]
        assert b.shape[1] == rank
        out = out_total - row_offset if out is None else out
        if staging is None:
            check(lib.sfq_lora_attach(self._h, C.c_void_p(key), a.ctypes.data, b.ctypes.data, rank, k, out_total, row_offset, out))
            return None
        host, device, offset = staging
        off = C.c_size_t(offset)
        check(lib.sfq_lora_attach_staged(self._h, C.c_void_p(key), a.ctypes.data, b.ctypes.data, rank, k, out_total, row_offset, out,
                                         C.c_void_p(host), C.c_void_p(device), C.byref(off)))
        return off.value

    def apply(self, key: int, x, y):
        """x: bf16 [rows, in] on the device; y: bf16 [rows, out], updated in place."""
        check(lib.sfq_lora_apply(self._h, C.c_void_p(key), ptr(x), x.shape[0], ptr(y), stream_ptr()))
        return y

    def bytes(self):
        w, s = C.c_size_t(), C.c_size_t()
        check(lib.sfq_lora_bytes(self._h, C.byref(w), C.byref(s)))
        return w.value, s.value
