"""safetensors files for the quantized Linear: a writer for synthetic checkpoints in the reference's on-disk
conventions and a thin wrapper over the C reader (``sfq_checkpoint_*``).

File layout: u64 little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}, "__metadata__":
{...}}``, then the tensor bytes (the reference reads it in src/core/safetensors.cpp).
"""
from __future__ import annotations

import ctypes as C
import json
import struct

import numpy as np

from . import QuantWeight, check, lib

_NUMPY_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I8": np.int8, "U8": np.uint8, "I16": np.int16,
                 "I32": np.int32, "I64": np.int64, "BOOL": np.bool_}
DTYPE_NAMES = ["UNKNOWN", "BOOL", "U8", "I8", "I16", "I32", "I64", "F8_E4M3", "F8_E5M2", "F16", "BF16", "F32", "F64"]


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> numpy array, or (dtype name, shape, raw bytes / array) for types numpy lacks
    ("BF16" from uint16 bits, "F8_E4M3" from uint8 bits)."""
    header, blobs, offset = {}, [], 0
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, value in tensors.items():
        if isinstance(value, tuple):
            dtype, shape, raw = value
            raw = np.ascontiguousarray(raw).tobytes() if not isinstance(raw, (bytes, bytearray)) else bytes(raw)
        else:
            arr = np.ascontiguousarray(value)
            dtype = next(k for k, v in _NUMPY_DTYPES.items() if np.dtype(v) == arr.dtype)
            shape, raw = list(arr.shape), arr.tobytes()
        header[name] = {"dtype": dtype, "shape": [int(d) for d in shape], "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def json_tensor(obj) -> tuple:
    """A rank-1 U8 tensor holding JSON text, the form of ``.comfy_quant`` and the bitsandbytes state tensors."""
    raw = json.dumps(obj).encode()
    return ("U8", [len(raw)], raw)


class Checkpoint:
    def __init__(self, path: str):
        self._h = C.c_void_p()
        check(lib.sfq_checkpoint_open(path.encode(), C.byref(self._h)))

    def close(self) -> None:
        if self._h:
            lib.sfq_checkpoint_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self) -> int:
        return lib.sfq_checkpoint_count(self._h)

    def tensor(self, name: str):
        """(dtype name, shape, bytes as a uint8 numpy array copied out of the mapping)."""
        dtype, rank, nbytes = C.c_int32(), C.c_int32(), C.c_size_t()
        shape = (C.c_int64 * 8)()
        data = C.c_void_p()
        check(lib.sfq_checkpoint_tensor(self._h, name.encode(), C.byref(dtype), C.byref(rank), shape, C.byref(data), C.byref(nbytes)))
        raw = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nbytes.value,)).copy() if nbytes.value else np.zeros(0, np.uint8)
        return DTYPE_NAMES[dtype.value], [shape[i] for i in range(rank.value)], raw

    def metadata(self, key: str) -> str:
        n = C.c_size_t()
        check(lib.sfq_checkpoint_metadata(self._h, key.encode(), None, 0, C.byref(n)))
        buf = C.create_string_buffer(n.value + 1)
        check(lib.sfq_checkpoint_metadata(self._h, key.encode(), buf, n.value + 1, C.byref(n)))
        return buf.value.decode()

    def linear(self, name: str, out_features: int, in_features: int, host: bool = False) -> QuantWeight:
        """The layer's QuantWeight with device pointers (uploads on first use), or host pointers with host=True.
        The checkpoint must stay open while the weight is in use."""
        w = QuantWeight()
        fn = lib.sfq_checkpoint_linear_host if host else lib.sfq_checkpoint_linear
        check(fn(self._h, name.encode(), out_features, in_features, C.byref(w)))
        return w
