"""slopfab_b200 -- B200-native quantized Linear for slopfab's DiT.

The product is ``libsfq.so`` (hand-written sm_100a CUDA kernels, the C++
``slopfab::cuda::LinearRunner`` mirror and the C ABI of ``include/sfq.h``). This
package is the ctypes binding used by the tests and the benchmark: it passes
torch device pointers straight to the C ABI. There is no fallback path of any
kind: if the library is missing, importing :data:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsfq.so")

OK, ERR_INVALID_ARGUMENT, ERR_RUNTIME, ERR_OUT_OF_MEMORY, ERR_DEVICE_TIMEOUT = 0, -1, -2, -3, -4
F32, F16, BF16, F8E4M3, I8, NVFP4, NF4, W4A8, W6A8 = range(9)
COMPUTE_BF16, COMPUTE_F32 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_SWIGLU = 0, 1, 2
NVFP4_ACT_REFERENCE, NVFP4_ACT_GEMM_FEED = 0, 1

V, I, U32, F, SZ = C.c_void_p, C.c_int, C.c_uint32, C.c_float, C.c_size_t


class QuantWeight(C.Structure):
    """sfq_quant_weight (include/sfq.h), the C mirror of the reference's QuantWeight."""
    _fields_ = [("format", C.c_int32), ("data", V), ("out_features", C.c_int32), ("in_features", C.c_int32),
                ("weight_scale", V), ("per_channel_scale", C.c_int32), ("input_scale", F),
                ("full_precision", C.c_int32), ("block_scale", V), ("packed_group_size", U32),
                ("w4_codebook", V), ("global_scale", F), ("pre_quant_scale", V), ("nf4_absmax", V),
                ("nf4_quant_map", V), ("nf4_nested_quant_map", V), ("nf4_nested_absmax", V),
                ("nf4_block_size", C.c_int32), ("nf4_nested_block_size", C.c_int32), ("nf4_nested_offset", F),
                ("convrot", C.c_int32), ("convrot_group", C.c_int32), ("bias", V), ("bias_format", C.c_int32)]


class Epilogue(C.Structure):
    _fields_ = [("d_row_scale", V), ("d_col_scale", V), ("global_scale", F), ("d_bias", V),
                ("bias_format", C.c_int32), ("activation", C.c_int32), ("d_gate", V), ("d_gate_index", V)]


class Norm(C.Structure):
    _fields_ = [("d_norm_weight", V), ("d_scale", V), ("d_shift", V), ("d_adaln_index", V), ("eps", F)]


class SequenceLayout(C.Structure):
    _fields_ = [("num_text", C.c_int32), ("num_condition_video", C.c_int32), ("num_condition_audio", C.c_int32),
                ("condition_audio_is_explicit", C.c_int32), ("num_audio_rows", C.c_int32), ("num_video_rows", C.c_int32)]


class SfqError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"sfq error {code}: {message}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python slopfab_b200/build.py` "
                          "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    P = C.POINTER
    sigs = {
        "sfq_last_error": (C.c_char_p, []),
        "sfq_version": (I, []),
        "sfq_quant_weight_init": (None, [P(QuantWeight)]),
        "sfq_device_status": (I, [P(I)]),
        "sfq_pack_nvfp4": (I, [V, I, I, F, V, V]),
        "sfq_pack_w4a8": (I, [V, I, I, V, V, V, V]),
        "sfq_pack_w6a8": (I, [V, I, I, I, V, V, V]),
        "sfq_pack_int8": (I, [V, I, I, I, V, V]),
        "sfq_unpack_nvfp4_bf16": (I, [V, V, F, V, I, I, V]),
        "sfq_unpack_w4a8_int8": (I, [V, V, V, V, I, I, I, V]),
        "sfq_unpack_w6a8_int8": (I, [V, V, V, I, I, I, V]),
        "sfq_unpack_int8_bf16": (I, [V, V, V, I, I, V]),
        "sfq_unpack_int8_f16": (I, [V, V, V, I, I, I, I, V]),
        "sfq_unpack_f8e4m3_bf16": (I, [V, V, V, SZ, V]),
        "sfq_unpack_nf4_bf16": (I, [V, V, V, V, V, I, I, F, V, I, I, V]),
        "sfq_pre_quant_scale": (I, [V, V, V, I, I, V]),
        "sfq_rmsnorm": (I, [V, P(Norm), V, I, I, V]),
        "sfq_convrot": (I, [V, V, I, I, I, V]),
        "sfq_convrot_f32": (I, [V, V, I, I, I, V]),
        "sfq_int8_output_bf16": (I, [V, V, V, V, I, I, V]),
        "sfq_int8_output_f32": (I, [V, V, V, I, I, V]),
        "sfq_quantize_f8e4m3": (I, [V, F, V, SZ, V]),
        "sfq_unpack_nf4_f16": (I, [V, V, V, V, V, I, I, F, V, SZ, V]),
        "sfq_gemm_nvfp4_reference_layout": (I, [V, V, V, V, F, V, I, I, I, V]),
        "sfq_quantize_int8_token": (I, [V, P(Norm), V, V, V, I, I, I, V]),
        "sfq_quantize_nvfp4_block": (I, [V, P(Norm), V, V, V, I, I, I, V]),
        "sfq_nvfp4_act_scale_bytes": (SZ, [I, I]),
        "sfq_gelu_tanh": (I, [V, SZ, V]),
        "sfq_swiglu": (I, [V, V, I, I, V]),
        "sfq_add_gated": (I, [V, V, V, V, I, I, V]),
        "sfq_gemm_int8": (I, [V, V, P(Epilogue), V, I, I, I, V]),
        "sfq_gemm_w4a8_fused": (I, [V, V, V, V, P(Epilogue), V, I, I, I, V]),
        "sfq_gemm_nvfp4": (I, [V, V, V, V, P(Epilogue), V, I, I, I, V]),
        "sfq_gemm_bf16": (I, [V, V, P(Epilogue), V, I, I, I, V]),
        "sfq_test_gemm_variant": (None, [I, I, I]),
        "sfq_test_gemm_lost_load": (None, [I, C.c_longlong]),
        "sfq_runner_create": (I, [V, P(V)]),
        "sfq_runner_destroy": (None, [V]),
        "sfq_runner_set_native": (I, [V, I]),
        "sfq_runner_native": (I, [V]),
        "sfq_runner_set_activation": (I, [V, I]),
        "sfq_linear_workspace_bytes": (I, [P(QuantWeight), I, I, P(SZ)]),
        "sfq_linear_dense_weight_bytes": (I, [P(QuantWeight), P(SZ)]),
        "sfq_linear_activation_workspace_bytes": (I, [P(QuantWeight), I, I, P(SZ)]),
        "sfq_linear_forward": (I, [V, P(QuantWeight), V, I, V, V, SZ]),
        "sfq_linear_prepare": (I, [V, P(QuantWeight), V, SZ, P(V), P(SZ)]),
        "sfq_linear_forward_prepared": (I, [V, P(QuantWeight), V, V, I, V, V, SZ]),
        "sfq_linear_nvfp4_forward_static": (I, [V, I, V, V, F, V, I, I, V, I, I, V]),
        "sfq_static_status": (I, [P(I)]),
        "sfq_build_indices": (I, [P(SequenceLayout), V, V, V, V]),
        "sfq_build_row_timesteps": (I, [P(SequenceLayout), V, F, F, V, V, V, I, P(I)]),
        "sfq_build_row_timesteps4": (I, [P(SequenceLayout), V, F, F, F, F, V, V, V, I, P(I)]),
        "sfq_build_adaln_index": (I, [I, I, I, I, I, I, F, F, V, V, V, V, P(I)]),
        "sfq_weight_row_block": (I, [P(QuantWeight), I, I, P(QuantWeight)]),
        "sfq_checkpoint_open": (I, [C.c_char_p, P(V)]),
        "sfq_checkpoint_close": (None, [V]),
        "sfq_checkpoint_count": (I, [V]),
        "sfq_checkpoint_tensor": (I, [V, C.c_char_p, P(C.c_int32), P(C.c_int32), P(C.c_int64), P(V), P(SZ)]),
        "sfq_checkpoint_metadata": (I, [V, C.c_char_p, C.c_char_p, SZ, P(SZ)]),
        "sfq_checkpoint_linear": (I, [V, C.c_char_p, I, I, P(QuantWeight)]),
        "sfq_checkpoint_linear_host": (I, [V, C.c_char_p, I, I, P(QuantWeight)]),
        "sfq_linear_forward_f32": (I, [V, P(QuantWeight), V, I, V, V, SZ]),
        "sfq_adaln_expand": (I, [V, V, V, V, I, I, I, I, I, V]),
        "sfq_head_norm_rope": (I, [V, I, V, V, V, I, I, I, C.c_float, V]),
        "sfq_attention_workspace_bytes": (I, [I, I, I, P(SZ)]),
        "sfq_attention_forward": (I, [V, I, V, V, I, V, I, I, I, I, I, I, C.c_float, V, SZ, V]),
        "sfq_lora_create": (I, [P(V)]),
        "sfq_lora_destroy": (None, [V]),
        "sfq_lora_attach": (I, [V, V, V, V, I, I, I, I, I]),
        "sfq_lora_attach_staged": (I, [V, V, V, V, I, I, I, I, I, V, V, P(SZ)]),
        "sfq_lora_apply": (I, [V, V, V, I, V, V]),
        "sfq_lora_bytes": (I, [V, P(SZ), P(SZ)]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
EXPORTS = ("sfq_last_error sfq_version sfq_quant_weight_init sfq_device_status sfq_pack_nvfp4 sfq_pack_w4a8 "
           "sfq_pack_w6a8 sfq_pack_int8 sfq_unpack_nvfp4_bf16 sfq_unpack_w4a8_int8 sfq_unpack_w6a8_int8 "
           "sfq_unpack_int8_bf16 sfq_unpack_int8_f16 sfq_unpack_f8e4m3_bf16 sfq_unpack_nf4_bf16 sfq_pre_quant_scale sfq_rmsnorm sfq_convrot sfq_convrot_f32 sfq_int8_output_bf16 sfq_int8_output_f32 sfq_quantize_f8e4m3 sfq_unpack_nf4_f16 sfq_gemm_nvfp4_reference_layout sfq_quantize_int8_token "
           "sfq_quantize_nvfp4_block sfq_nvfp4_act_scale_bytes sfq_gelu_tanh sfq_swiglu sfq_add_gated sfq_gemm_int8 sfq_gemm_w4a8_fused "
           "sfq_gemm_nvfp4 sfq_gemm_bf16 sfq_test_gemm_variant sfq_test_gemm_lost_load sfq_runner_create sfq_runner_destroy sfq_runner_set_native "
           "sfq_runner_native sfq_runner_set_activation sfq_linear_workspace_bytes sfq_linear_dense_weight_bytes "
           "sfq_linear_activation_workspace_bytes sfq_linear_forward sfq_linear_prepare "
           "sfq_linear_forward_prepared sfq_linear_nvfp4_forward_static sfq_static_status sfq_build_indices sfq_build_row_timesteps sfq_build_row_timesteps4 sfq_build_adaln_index sfq_weight_row_block sfq_checkpoint_open "
           "sfq_checkpoint_close sfq_checkpoint_count sfq_checkpoint_tensor sfq_checkpoint_metadata sfq_checkpoint_linear sfq_checkpoint_linear_host "
           "sfq_linear_forward_f32 sfq_adaln_expand sfq_head_norm_rope sfq_attention_workspace_bytes sfq_attention_forward sfq_lora_create sfq_lora_destroy sfq_lora_attach sfq_lora_attach_staged sfq_lora_apply sfq_lora_bytes").split()
STATIC_SCRATCH_BYTES = 16 * 1024 * 1024


def check(status: int) -> None:
    if status != OK:
        raise SfqError(status, lib.sfq_last_error().decode("utf-8", "replace"))


def device_status() -> int:
    """Reads and clears the device status word (synchronises). Non-zero = a kernel gave up a bounded wait."""
    code = I(0)
    check(lib.sfq_device_status(C.byref(code)))
    return code.value


def static_status() -> int:
    """Reads and clears the status word of sfq_linear_nvfp4_forward_static (its kernels do not write the word above)."""
    code = I(0)
    check(lib.sfq_static_status(C.byref(code)))
    return code.value


def ptr(t) -> int | None:
    """Device (or host) address of a torch tensor / numpy array, None for None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        assert t.is_contiguous(), "sfq expects contiguous tensors"
        return t.data_ptr()
    assert t.flags["C_CONTIGUOUS"]
    return t.ctypes.data


def new_weight(**fields) -> QuantWeight:
    w = QuantWeight()
    lib.sfq_quant_weight_init(C.byref(w))
    for k, v in fields.items():
        setattr(w, k, v)
    return w


from .linear import LinearRunner, stream_ptr  # noqa: E402,F401
