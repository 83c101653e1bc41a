"""Shared helpers of the GPU parity tests: bf16 bit views, seeded inputs with the benchmark
configurations' distributions, packed weights, and typed access to the compiled reference."""
import ctypes as C

import numpy as np
import torch

import oracle
import slopfab_b200 as sfq

P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16/fp16 CUDA tensor -> uint16 numpy bits."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bf16_tensor(bits_u16: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits_u16).view(np.int16)).view(torch.bfloat16).to(device)


def dev(a: np.ndarray, device="cuda") -> torch.Tensor:
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(device)
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def gaussian_bf16(shape, seed, sigma=1.0, outliers=False) -> np.ndarray:
    rng = np.random.default_rng(seed)
    x = (sigma * rng.standard_normal(shape)).astype(np.float32)
    if outliers:  # 0.1 % of the elements x20
        mask = rng.random(shape) < 1e-3
        x = np.where(mask, x * 20.0, x).astype(np.float32)
    return oracle.to_bf16(x)


def pack_nvfp4(w: np.ndarray):
    n, k = w.shape
    g = float(np.abs(w).max() / (6.0 * 448.0))
    data = np.zeros((n, k // 2), np.uint8)
    scale = np.zeros(n * k // 16, np.uint8)
    sfq.check(sfq.lib.sfq_pack_nvfp4(P(np.ascontiguousarray(w, np.float32)), n, k, g, P(data), P(scale)))
    return data, scale, g


def pack_w4a8(w: np.ndarray):
    n, k = w.shape
    packed = np.zeros((n, k // 2), np.int8)
    s_rel = np.zeros(n * k // 16, np.uint8)
    s_ch = np.zeros(n, np.float32)
    book = np.zeros(16, np.float32)
    sfq.check(sfq.lib.sfq_pack_w4a8(P(np.ascontiguousarray(w, np.float32)), n, k, P(packed), P(s_rel), P(s_ch), P(book)))
    return packed, s_rel, s_ch, book


def pack_w6a8(w: np.ndarray, group: int):
    n, k = w.shape
    packed = np.zeros((n, k * 3 // 4), np.int8)
    s_rel = np.zeros(n * k // group, np.uint8)
    s_ch = np.zeros(n, np.float32)
    sfq.check(sfq.lib.sfq_pack_w6a8(P(np.ascontiguousarray(w, np.float32)), n, k, group, P(packed), P(s_rel), P(s_ch)))
    return packed, s_rel, s_ch


def synthetic_packed_int8(bits_: int, group: int, n: int, k: int, seed: int):
    """Random codes / scale bytes / channel scales straight in storage form (fast; no encoder)."""
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 256, size=(n, k * bits_ // 8), dtype=np.uint8).view(np.int8)
    s_rel = rng.choice(np.array([0x28, 0x2C, 0x30, 0x34, 0x38], np.uint8), size=n * k // group)
    s_ch = (2.0 ** rng.integers(-9, -5, size=n)).astype(np.float32) * (1 + rng.random(n).astype(np.float32))
    book = (np.arange(16, dtype=np.float32) - 8.0) if bits_ == 4 else None
    return packed, s_rel, s_ch.astype(np.float32), book


class RefWeight(C.Structure):
    _fields_ = [("format", C.c_int), ("data", C.c_void_p), ("out_features", C.c_int), ("in_features", C.c_int),
                ("weight_scale", C.c_void_p), ("per_channel_scale", C.c_int), ("block_scale", C.c_void_p),
                ("packed_group_size", C.c_uint32), ("w4_codebook", C.c_void_p), ("global_scale", C.c_float),
                ("convrot", C.c_int), ("convrot_group", C.c_int), ("bias", C.c_void_p), ("bias_format", C.c_int),
                ("pre_quant_scale", C.c_void_p), ("nf4_absmax", C.c_void_p), ("nf4_quant_map", C.c_void_p),
                ("nf4_nested_quant_map", C.c_void_p), ("nf4_nested_absmax", C.c_void_p), ("nf4_block_size", C.c_int),
                ("nf4_nested_block_size", C.c_int), ("nf4_nested_offset", C.c_float)]


def ref_weight_from(w: sfq.QuantWeight) -> RefWeight:
    r = RefWeight()
    for name, _ in RefWeight._fields_:
        setattr(r, name, getattr(w, name))
    return r


def ref_dev():
    """The compiled reference with its device entry points typed, or None."""
    ref = oracle.ref
    if ref is None:
        return None
    V, I, F, SZ = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    sigs = {"ref_dev_dequant_nvfp4": [V, V, F, V, I, I], "ref_dev_dequant_i8": [V, V, V, I, I],
            "ref_dev_dequant_w4a8": [V, V, V, V, I, I, I], "ref_dev_dequant_w6a8": [V, V, V, I, I, I],
            "ref_dev_dequant_f8": [V, V, V, SZ], "ref_dev_dequant_nf4": [V, V, V, V, V, I, I, F, V, I, I],
            "ref_dev_pre_quant_scale": [V, V, V, I, I], "ref_dev_convrot": [V, V, I, I, I], "ref_dev_quantize_int8_bf16": [V, V, V, I, I],
            "ref_dev_quantize_int8_f16": [V, V, V, I, I], "ref_dev_output_bf16": [V, V, V, V, I, I],
            "ref_dev_quantize_nvfp4_act": [V, V, V, I, I], "ref_dev_rmsnorm": [V, V, V, V, V, V, I, I, F],
            "ref_dev_gelu_tanh": [V, SZ], "ref_dev_swiglu": [V, V, I, I], "ref_dev_add_gated": [V, V, V, V, I, I],
            "ref_dev_linear_forward": [C.POINTER(RefWeight), V, I, V, I, I, C.POINTER(F)],
            "ref_dev_packed_int8_accumulate": [C.POINTER(RefWeight), V, I, V, V, V, V, V],
            "ref_dev_convrot_f32": [V, V, I, I, I], "ref_dev_quantize_f8": [V, F, V, SZ],
            "ref_dev_dequant_nf4_f16": [V, V, V, V, V, I, I, F, V, SZ], "ref_dev_output_f32": [V, V, V, I, I],
            "ref_dev_linear_forward_f32": [C.POINTER(RefWeight), V, I, V]}
    for name, args in sigs.items():
        fn = getattr(ref, name)
        fn.restype = I
        fn.argtypes = args
    ref.ref_last_error.restype = C.c_char_p
    return ref


def ref_check(ref, status):
    assert status == 0, ref.ref_last_error().decode()
