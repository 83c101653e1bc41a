"""numpy front end of the CPU oracle and of the compiled reference.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
`cpu_baseline` / `--impl reference` legs of bench.py, never by the product
package. bf16 and fp16 tensors travel as ``uint16`` arrays.

``lib``  -- oracle/liboracle.so, the CPU restatement (oracle/oracle.cpp).
``ref``  -- oracle/_ref/libslopfab_ref.so, the reference's own sources compiled
            in place (oracle/ref_shim.cu), or ``None`` when it was not built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libslopfab_ref.so")


def reference_root() -> str | None:
    """Root of the reference tree: $SLOPFAB_REFERENCE, else a directory named `reference` beside this repository;
    None when neither exists (the GPU box: only the prebuilt oracle/_ref travels there)."""
    for cand in (os.environ.get("SLOPFAB_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "cuda")):
            return cand
    return None


def build(with_reference: bool = True) -> None:
    """Compile the checkers (oracle always; the reference when its tree is present)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    root = reference_root() if with_reference else None
    if root is not None:
        subprocess.run(["make", "-C", _HERE, "-j8", "ref", "REF=" + root], check=True, capture_output=True)


if not os.path.exists(_LIB_PATH):
    build(with_reference=False)
lib = C.CDLL(_LIB_PATH)
ref = C.CDLL(_REF_PATH) if os.path.exists(_REF_PATH) else None

u8p, i8p, u16p, i32p, f32p = (C.POINTER(t) for t in (C.c_uint8, C.c_int8, C.c_uint16, C.c_int32, C.c_float))


def _p(a, ty=C.c_void_p):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ty)


def _sig(fn, res, *args):
    fn.restype = res
    fn.argtypes = list(args)


V = C.c_void_p
_sig(lib.orc_f32_to_bf16, C.c_uint16, C.c_float)
_sig(lib.orc_bf16_to_f32, C.c_float, C.c_uint16)
_sig(lib.orc_f32_to_f16, C.c_uint16, C.c_float)
_sig(lib.orc_f16_to_f32, C.c_float, C.c_uint16)
_sig(lib.orc_e4m3_to_f32, C.c_float, C.c_uint8)
_sig(lib.orc_f32_to_e4m3, C.c_uint8, C.c_float)
_sig(lib.orc_e4m3_nearest_nonneg, C.c_uint8, C.c_float)
_sig(lib.orc_e2m1_to_f32, C.c_float, C.c_uint8)
_sig(lib.orc_f32_to_e2m1, C.c_uint8, C.c_float)
_sig(lib.orc_nvfp4_scale_slot, C.c_uint64, C.c_int, C.c_int, C.c_int)
_sig(lib.orc_norm_rsqrt, C.c_float, C.c_float, C.c_uint32, C.c_float)
_sig(lib.orc_rsqrt_q30, C.c_float, C.c_float)
_sig(lib.orc_f32_to_bf16_n, None, V, V, C.c_size_t)
_sig(lib.orc_bf16_to_f32_n, None, V, V, C.c_size_t)
_sig(lib.orc_make_data, None, V, C.c_size_t, C.c_uint32, C.c_float)
_sig(lib.orc_make_gaussian, None, V, C.c_size_t, C.c_uint32, C.c_float)
_sig(lib.orc_nvfp4_pack, None, V, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, V, V, V)
_sig(lib.orc_nvfp4_dequant_bf16, None, V, V, C.c_float, C.c_int, C.c_int, V)
_sig(lib.orc_nvfp4_quantize_act, None, V, C.c_int, C.c_int, V, V, V)
_sig(lib.orc_w4a8_decode, None, V, V, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_w6a8_decode, None, V, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_int8_dequant_bf16, None, V, V, C.c_int, C.c_int, V)
_sig(lib.orc_int8_unpack_f16, None, V, V, C.c_int, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_f8_dequant_bf16, None, V, C.c_float, C.c_size_t, V)
_sig(lib.orc_nf4_dequant_bf16, None, V, V, V, V, V, C.c_int, C.c_int, C.c_float, C.c_size_t, V)
_sig(lib.orc_f16_to_bf16_n, None, V, V, C.c_size_t)
_sig(lib.orc_pre_quant_scale_bf16, None, V, V, C.c_int, C.c_int, V)
_sig(lib.orc_convrot_bf16, None, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_convrot_dense_f32, None, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_quantize_int8_token, None, V, C.c_int, C.c_int, V, V)
_sig(lib.orc_quantize_int8_token_f16, None, V, C.c_int, C.c_int, V, V)
_sig(lib.orc_int8_gemm, None, V, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_w4a8_output_bf16, None, V, V, V, C.c_int, C.c_int, V)
_sig(lib.orc_add_bias_bf16, None, V, V, C.c_int, C.c_int, C.c_int)
_sig(lib.orc_gelu_tanh_bf16, None, V, C.c_size_t)
_sig(lib.orc_swiglu_bf16, None, V, C.c_int, C.c_int, V)
_sig(lib.orc_head_norm_rope, None, V, C.c_int, V, V, V, C.c_int, C.c_int, C.c_float)
_sig(lib.orc_attention, None, V, V, V, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, V)
_sig(lib.orc_adaln_expand, None, V, V, V, V, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int)
_sig(lib.orc_lora_apply, None, V, C.c_int, V, V, C.c_int, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_add_gated_bf16, None, V, V, V, V, C.c_int, C.c_int)
_sig(lib.orc_rmsnorm_bf16, None, V, V, V, V, V, C.c_int, C.c_int, C.c_float, V)
_sig(lib.orc_rmsnorm_spec_f32, None, V, V, V, V, V, C.c_int, C.c_int, C.c_float, V)
_sig(lib.orc_matmul_nt, None, V, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_matmul_nt_fast, None, V, V, C.c_int, C.c_int, C.c_int, V)
_sig(lib.orc_num_threads, C.c_int)
_sig(lib.orc_set_num_threads, None, C.c_int)
_sig(lib.orc_nvfp4_linear, None, V, C.c_int, V, V, C.c_float, C.c_int, C.c_int, V, C.c_int, V)
_sig(lib.orc_nvfp4_linear_dequant, None, V, C.c_int, V, V, C.c_float, C.c_int, C.c_int, V, V)
_sig(lib.orc_packed_int8_linear, None, V, C.c_int, V, V, V, V, C.c_int, C.c_int, C.c_int, C.c_int,
     V, C.c_int, C.c_int, V, V, V, V, V, V)
_sig(lib.orc_host_dequant_matmul, None, C.c_int, V, C.c_int, V, V, V, V, C.c_float, C.c_int, C.c_int,
     C.c_int, V)
_sig(lib.orc_compare_bf16, None, V, V, C.c_size_t, V)

ACT_NONE, ACT_GELU_TANH = 0, 1


# --------------------------------------------------------------------------- conversions
def to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib.orc_f32_to_bf16_n(_p(x), _p(out), x.size)
    return out


def from_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib.orc_bf16_to_f32_n(_p(x), _p(out), x.size)
    return out


def make_data(n: int, seed: int, scale: float) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib.orc_make_data(_p(out), n, seed, scale)
    return out


def make_gaussian(n: int, seed: int, sigma: float) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib.orc_make_gaussian(_p(out), n, seed, sigma)
    return out


# --------------------------------------------------------------------------- nvfp4
def nvfp4_pack(w: np.ndarray, global_scale: float, high_even=True, swizzled=True):
    """fp32 [N,K] -> (data u8 [N,K/2], scale u8 [N*K/16], dense f32 [N,K])."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    data = np.zeros((n, k // 2), np.uint8)
    scale = np.zeros(n * k // 16, np.uint8)
    dense = np.zeros((n, k), np.float32)
    lib.orc_nvfp4_pack(_p(w), n, k, global_scale, int(high_even), int(swizzled), _p(data), _p(scale), _p(dense))
    return data, scale, dense


def nvfp4_dequant_bf16(data, scale, global_scale, n, k):
    out = np.empty((n, k), np.uint16)
    lib.orc_nvfp4_dequant_bf16(_p(data), _p(scale), global_scale, n, k, _p(out))
    return out


def nvfp4_quantize_act(x_bf16: np.ndarray):
    """bf16 [M,K] -> (packed u8 [M,K/2] low-nibble-even, scales u8 [M,K/16], dense f32)."""
    m, k = x_bf16.shape
    packed = np.empty((m, k // 2), np.uint8)
    scales = np.empty((m, k // 16), np.uint8)
    dense = np.empty((m, k), np.float32)
    lib.orc_nvfp4_quantize_act(_p(x_bf16), m, k, _p(packed), _p(scales), _p(dense))
    return packed, scales, dense


def nvfp4_linear(x_bf16, wdata, wscale, global_scale, n, k, bias=None, act=ACT_NONE):
    m = x_bf16.shape[0]
    y = np.empty((m, n), np.uint16)
    lib.orc_nvfp4_linear(_p(x_bf16), m, _p(wdata), _p(wscale), global_scale, n, k, _p(bias), act, _p(y))
    return y


def nvfp4_linear_dequant(x_bf16, wdata, wscale, global_scale, n, k, bias=None):
    m = x_bf16.shape[0]
    y = np.empty((m, n), np.uint16)
    lib.orc_nvfp4_linear_dequant(_p(x_bf16), m, _p(wdata), _p(wscale), global_scale, n, k, _p(bias), _p(y))
    return y


# --------------------------------------------------------------------------- packed int8
def w4a8_decode(packed, s_rel, codebook, n, k, group=16):
    out = np.empty((n, k), np.int8)
    lib.orc_w4a8_decode(_p(packed), _p(s_rel), _p(codebook), n, k, group, _p(out))
    return out


def w6a8_decode(packed, s_rel, n, k, group):
    out = np.empty((n, k), np.int8)
    lib.orc_w6a8_decode(_p(packed), _p(s_rel), n, k, group, _p(out))
    return out


def convrot_bf16(x_bf16, group=256):
    m, k = x_bf16.shape
    out = np.empty((m, k), np.uint16)
    lib.orc_convrot_bf16(_p(x_bf16), m, k, group, _p(out))
    return out


def convrot_dense(x_f32, group=256):
    x_f32 = np.ascontiguousarray(x_f32, np.float32)
    m, k = x_f32.shape
    out = np.empty((m, k), np.float32)
    lib.orc_convrot_dense_f32(_p(x_f32), m, k, group, _p(out))
    return out


def quantize_int8_token(x_bf16):
    m, k = x_bf16.shape
    q = np.empty((m, k), np.int8)
    s = np.empty(m, np.float32)
    lib.orc_quantize_int8_token(_p(x_bf16), m, k, _p(q), _p(s))
    return q, s


def int8_gemm(a, w):
    m, k = a.shape
    n = w.shape[0]
    acc = np.empty((m, n), np.int32)
    lib.orc_int8_gemm(_p(a), _p(w), m, n, k, _p(acc))
    return acc


def packed_int8_linear(x_bf16, packed, s_rel, s_channel, codebook, bits, group, n, k, bias=None,
                       bias_is_bf16=False, act=ACT_NONE, want_intermediates=False):
    m = x_bf16.shape[0]
    y = np.empty((m, n), np.uint16)
    inter = None
    if want_intermediates:
        inter = dict(w8=np.empty((n, k), np.int8), rot=np.empty((m, k), np.uint16),
                     q=np.empty((m, k), np.int8), row_scale=np.empty(m, np.float32),
                     acc=np.empty((m, n), np.int32))
    g = (lambda key: _p(inter[key])) if inter else (lambda key: None)
    lib.orc_packed_int8_linear(_p(x_bf16), m, _p(packed), _p(s_rel), _p(s_channel), _p(codebook), bits, group,
                               n, k, _p(bias), int(bias_is_bf16), act, _p(y), g("w8"), g("rot"), g("q"),
                               g("row_scale"), g("acc"))
    return (y, inter) if want_intermediates else y


def head_norm_rope(x_bf16, heads, w_bf16=None, cos=None, sin=None, eps=1e-6):
    """QK-norm then MM-RoPE on bf16 bits x [rows, >= heads*128] (row pitch = x.shape[1]); returns the new array."""
    x = np.array(x_bf16, np.uint16, copy=True)
    lib.orc_head_norm_rope(_p(x), x.shape[1], _p(w_bf16), _p(cos), _p(sin), x.shape[0], heads, eps)
    return x


def attention(q, k, v, heads, kv_heads, head_dim, scale):
    """Dense fp64 softmax attention on fp32 arrays q [seq_q, heads*dim], k / v [seq_kv, kv_heads*dim]."""
    q, k, v = (np.ascontiguousarray(t, np.float32) for t in (q, k, v))
    out = np.empty_like(q)
    lib.orc_attention(_p(q), _p(k), _p(v), q.shape[0], k.shape[0], heads, kv_heads, head_dim, scale, _p(out))
    return out


def adaln_expand(w, bias, code, num_modality, num_param, channels):
    """Modulation tables [param, t, modality, channel] (fp32) from w [features, rank], bias [features], code [t, rank]."""
    num_t, rank = code.shape
    out = np.empty((num_param, num_t, num_modality, channels), np.float32)
    lib.orc_adaln_expand(_p(np.ascontiguousarray(w, np.float32)), _p(np.ascontiguousarray(bias, np.float32)),
                         _p(np.ascontiguousarray(code, np.float32)), _p(out), num_t, num_modality, num_param, channels, rank)
    return out


def lora_apply(x_bf16, a, b, offset, out, y_bf16):
    """y += (x A^T) B[offset:offset+out]^T with the reference test's rounding points; returns the new y."""
    rows, k = x_bf16.shape
    rank = a.shape[0]
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    y = np.array(y_bf16, np.uint16, copy=True)
    lib.orc_lora_apply(_p(x_bf16), rows, _p(a), _p(b), rank, k, offset, out, _p(y))
    return y


# --------------------------------------------------------------------------- norm
def rmsnorm_bf16(x_bf16, w_bf16, eps, scale=None, shift=None, a=None):
    m, k = x_bf16.shape
    out = np.empty((m, k), np.uint16)
    lib.orc_rmsnorm_bf16(_p(x_bf16), _p(w_bf16), _p(scale), _p(shift), _p(a), m, k, eps, _p(out))
    return out


def compare_bf16(ref_bits, got_bits):
    """(max_abs, rel_l2, correlation) with the reference's metric definitions."""
    out = np.zeros(3, np.float64)
    r = np.ascontiguousarray(ref_bits, np.uint16)
    g = np.ascontiguousarray(got_bits, np.uint16)
    lib.orc_compare_bf16(_p(r), _p(g), r.size, _p(out))
    return float(out[0]), float(out[1]), float(out[2])
