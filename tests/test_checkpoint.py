"""The checkpoint boundary: safetensors parsing and the per-layer format rule (quant() of the reference's loader,
src/dit/transformer_load.cpp:585-659), on synthetic files written in the reference's on-disk conventions. Host-side:
the device upload and a forward from a loaded layer are in test_gpu_checkpoint.py."""
import ctypes as C
import json
import os
import struct

import numpy as np
import pytest

import oracle
import slopfab_b200 as sfq
from slopfab_b200.checkpoint import Checkpoint, json_tensor, write_safetensors

OUT, IN = 256, 512


def host_bytes(ptr, n):
    return np.frombuffer(C.string_at(ptr, n), np.uint8)


def synthetic_layers(rng):
    """One layer per storage format, named like the DiT's projections."""
    n = OUT * IN
    t, truth = {}, {}
    # W4A8: nibbles, e4m3 group scales, fp32 channel scales, fp32 codebook; tag in <layer>.comfy_quant
    truth["blocks.0.attn.out_proj"] = dict(format=sfq.W4A8)
    t["blocks.0.attn.out_proj.weight"] = ("U8", [OUT, IN // 2], rng.integers(0, 256, n // 2, dtype=np.uint8))
    t["blocks.0.attn.out_proj.weight_s_rel"] = ("F8_E4M3", [OUT, IN // 16], rng.integers(0x28, 0x40, n // 16, dtype=np.uint8))
    t["blocks.0.attn.out_proj.weight_s_channel"] = rng.random(OUT, dtype=np.float32)
    t["blocks.0.attn.out_proj.weight_codebook"] = np.arange(16, dtype=np.float32) - 8
    t["blocks.0.attn.out_proj.comfy_quant"] = json_tensor({"format": "asym_w4a8_int8", "group_size": 16, "convrot": True,
                                                          "convrot_groupsize": 256})
    # W6A8, group 64, parameters under "params"
    t["blocks.0.mlp.fc2.weight"] = ("U8", [OUT, IN * 3 // 4], rng.integers(0, 256, n * 3 // 4, dtype=np.uint8))
    t["blocks.0.mlp.fc2.weight_s_rel"] = ("F8_E4M3", [OUT, IN // 64], rng.integers(0x28, 0x40, n // 64, dtype=np.uint8))
    t["blocks.0.mlp.fc2.weight_s_channel"] = ("BF16", [OUT], (rng.integers(0x3C00, 0x3F00, OUT)).astype(np.uint16))
    t["blocks.0.mlp.fc2.comfy_quant"] = json_tensor({"format": "w6a8_int8", "params": {"group_size": 64, "convrot_groupsize": 256}})
    # NVFP4: U8 nibbles + e4m3 [N, K/16] scales + fp32 scalar
    t["blocks.1.attn.out_proj.weight"] = ("U8", [OUT, IN // 2], rng.integers(0, 256, n // 2, dtype=np.uint8))
    t["blocks.1.attn.out_proj.weight_scale"] = ("F8_E4M3", [OUT, IN // 16], rng.integers(0x30, 0x40, n // 16, dtype=np.uint8))
    t["blocks.1.attn.out_proj.weight_scale_2"] = np.array([0.0125], np.float32)
    t["blocks.1.attn.out_proj.input_scale"] = np.array([0.5], np.float32)
    # NF4 with bitsandbytes double quantization
    t["blocks.2.attn.out_proj.weight"] = ("U8", [n // 2, 1], rng.integers(0, 256, n // 2, dtype=np.uint8))
    t["blocks.2.attn.out_proj.weight.absmax"] = rng.integers(0, 256, n // 64, dtype=np.uint8)
    t["blocks.2.attn.out_proj.weight.quant_map"] = np.linspace(-1, 1, 16, dtype=np.float32)
    t["blocks.2.attn.out_proj.weight.nested_absmax"] = rng.random(n // 64 // 256, dtype=np.float32)
    t["blocks.2.attn.out_proj.weight.nested_quant_map"] = np.linspace(-1, 1, 256, dtype=np.float32)
    t["blocks.2.attn.out_proj.weight.quant_state.bitsandbytes__nf4"] = json_tensor(
        {"quant_type": "nf4", "nested_dtype": "float32", "dtype": "bfloat16", "blocksize": 64, "nested_blocksize": 256,
         "nested_offset": 0.03, "shape": [OUT, IN]})
    # fp8 per tensor, int8 per channel with a ConvRot tag from the header table, bf16, f16, f32
    t["blocks.3.mlp.fc1.weight"] = ("F8_E4M3", [OUT, IN], rng.integers(0, 0x7E, n, dtype=np.uint8))
    t["blocks.3.mlp.fc1.weight_scale"] = np.array([0.02], np.float32)
    t["text.proj.weight"] = rng.integers(-127, 128, (OUT, IN), dtype=np.int8)
    t["text.proj.weight_scale"] = rng.random(OUT, dtype=np.float32)
    t["refiner.0.proj.weight"] = ("BF16", [OUT, IN], rng.integers(0, 0x4000, n).astype(np.uint16))
    t["vae.proj.weight"] = rng.standard_normal((OUT, IN)).astype(np.float16)
    t["time.proj.weight"] = rng.standard_normal((OUT, IN)).astype(np.float32)
    meta = {"_quantization_metadata": json.dumps({"format_version": "1.0", "layers": {
        "text.proj": {"format": "int8_tensorwise", "convrot": True, "convrot_groupsize": 64}}}), "producer": "synthetic"}
    return t, meta


@pytest.fixture(scope="module")
def checkpoint_path(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("ckpt") / "layers.safetensors")
    tensors, meta = synthetic_layers(np.random.default_rng(3))
    write_safetensors(path, tensors, meta)
    return path, tensors


def _raw(value):
    return np.ascontiguousarray(value[2] if isinstance(value, tuple) else value).view(np.uint8).reshape(-1)


def test_header_entries_and_metadata(checkpoint_path):
    path, tensors = checkpoint_path
    with Checkpoint(path) as ck:
        assert len(ck) == len(tensors)
        for name, value in tensors.items():
            dtype, shape, raw = ck.tensor(name)
            want_shape = value[1] if isinstance(value, tuple) else list(value.shape)
            assert shape == [int(d) for d in want_shape], name
            assert np.array_equal(raw, _raw(value)), name
        assert ck.tensor("blocks.0.mlp.fc2.weight_s_rel")[0] == "F8_E4M3"
        assert ck.tensor("refiner.0.proj.weight")[0] == "BF16"
        assert ck.metadata("producer") == "synthetic"
        with pytest.raises(sfq.SfqError):
            ck.tensor("no.such.tensor")


def test_layer_rule_for_every_format(checkpoint_path):
    path, tensors = checkpoint_path
    n = OUT * IN
    with Checkpoint(path) as ck:
        w = ck.linear("blocks.0.attn.out_proj", OUT, IN, host=True)
        assert (w.format, w.packed_group_size, w.convrot, w.convrot_group, w.per_channel_scale) == (sfq.W4A8, 16, 1, 256, 1)
        assert np.array_equal(host_bytes(w.data, n // 2), _raw(tensors["blocks.0.attn.out_proj.weight"]))
        assert np.array_equal(host_bytes(w.block_scale, n // 16), _raw(tensors["blocks.0.attn.out_proj.weight_s_rel"]))
        assert np.array_equal(host_bytes(w.weight_scale, 4 * OUT), _raw(tensors["blocks.0.attn.out_proj.weight_s_channel"]))
        assert np.array_equal(host_bytes(w.w4_codebook, 64).view(np.float32), np.arange(16, dtype=np.float32) - 8)

        w = ck.linear("blocks.0.mlp.fc2", OUT, IN, host=True)
        assert (w.format, w.packed_group_size, w.convrot, w.convrot_group) == (sfq.W6A8, 64, 1, 256) and not w.w4_codebook
        bf = _raw(tensors["blocks.0.mlp.fc2.weight_s_channel"]).view(np.uint16).astype(np.uint32) << 16
        assert np.array_equal(host_bytes(w.weight_scale, 4 * OUT).view(np.uint32), bf)  # bf16 scales widened to fp32

        w = ck.linear("blocks.1.attn.out_proj", OUT, IN, host=True)
        assert w.format == sfq.NVFP4 and w.global_scale == np.float32(0.0125) and w.input_scale == 0.5 and w.convrot == 0
        assert np.array_equal(host_bytes(w.block_scale, n // 16), _raw(tensors["blocks.1.attn.out_proj.weight_scale"]))

        w = ck.linear("blocks.2.attn.out_proj", OUT, IN, host=True)
        assert (w.format, w.nf4_block_size, w.nf4_nested_block_size) == (sfq.NF4, 64, 256)
        assert w.nf4_nested_offset == np.float32(0.03)
        assert np.array_equal(host_bytes(w.nf4_absmax, n // 64), _raw(tensors["blocks.2.attn.out_proj.weight.absmax"]))
        assert np.array_equal(host_bytes(w.nf4_nested_quant_map, 1024).view(np.float32), np.linspace(-1, 1, 256, dtype=np.float32))

        w = ck.linear("blocks.3.mlp.fc1", OUT, IN, host=True)
        assert w.format == sfq.F8E4M3 and w.per_channel_scale == 0
        assert host_bytes(w.weight_scale, 4).view(np.float32)[0] == np.float32(0.02)

        w = ck.linear("text.proj", OUT, IN, host=True)  # ConvRot-64 from the header's table
        assert (w.format, w.per_channel_scale, w.convrot, w.convrot_group) == (sfq.I8, 1, 1, 64)
        for name, fmt in (("refiner.0.proj", sfq.BF16), ("vae.proj", sfq.F16), ("time.proj", sfq.F32)):
            w = ck.linear(name, OUT, IN, host=True)
            assert w.format == fmt and not w.weight_scale and w.convrot == 0
        # a layer whose sizes do not match the request is refused
        with pytest.raises(sfq.SfqError):
            ck.linear("time.proj", OUT, IN * 2, host=True)


def _refused(tmp_path, tensors, layer, meta=None, message=None):
    path = str(tmp_path / "bad.safetensors")
    write_safetensors(path, tensors, meta)
    with Checkpoint(path) as ck, pytest.raises(sfq.SfqError) as e:
        ck.linear(layer, OUT, IN, host=True)
    if message:
        assert message in str(e.value)


def test_refusals_of_the_reference_loader(tmp_path):
    rng = np.random.default_rng(5)
    n = OUT * IN
    nv = {"l.weight": ("U8", [OUT, IN // 2], rng.integers(0, 256, n // 2, dtype=np.uint8)),
          "l.weight_scale": ("F8_E4M3", [OUT, IN // 16], rng.integers(0x30, 0x40, n // 16, dtype=np.uint8))}
    _refused(tmp_path, nv, "l", message="weight_scale_2")                                 # nvfp4 without its tensor scale
    f8 = {"l.weight": ("F8_E4M3", [OUT, IN], rng.integers(0, 0x70, n, dtype=np.uint8))}
    _refused(tmp_path, f8, "l", message="fp8")
    i8 = {"l.weight": rng.integers(-127, 128, (OUT, IN), dtype=np.int8)}
    _refused(tmp_path, i8, "l", message="int8")
    w4 = {"l.weight": ("U8", [OUT, IN // 2], rng.integers(0, 256, n // 2, dtype=np.uint8)),
          "l.weight_s_rel": ("F8_E4M3", [OUT, IN // 16], rng.integers(0x28, 0x40, n // 16, dtype=np.uint8)),
          "l.weight_s_channel": rng.random(OUT, dtype=np.float32), "l.weight_codebook": np.arange(16, dtype=np.float32)}
    for tag in ({"format": "asym_w4a8_int8", "group_size": 32, "convrot_groupsize": 256},      # W4 needs group 16
                {"format": "asym_w4a8_int8", "group_size": 16, "convrot_groupsize": 64},       # ConvRot must be 256
                {"format": "asym_w4a8_int8", "group_size": 16, "convrot_groupsize": 256, "convrot": False},
                {"format": "asym_w4a8_int8", "group_size": 16},                                # incomplete state
                {"format": "some_future_format"}):
        _refused(tmp_path, dict(w4, **{"l.comfy_quant": json_tensor(tag)}), "l")
    # an int8 weight whose tag asks for a rotation group that is not a power of four
    bad_rot = dict(i8, **{"l.weight_scale": rng.random(OUT, dtype=np.float32),
                          "l.comfy_quant": json_tensor({"format": "int8_tensorwise", "convrot": True, "convrot_groupsize": 32})})
    _refused(tmp_path, bad_rot, "l", message="ConvRot")
    # a header table of an unknown version
    _refused(tmp_path, i8, "l", meta={"_quantization_metadata": json.dumps({"format_version": "2.0", "layers": {}})})
    # NF4 with a block size other than 64
    nf4 = {"l.weight": ("U8", [n // 2, 1], rng.integers(0, 256, n // 2, dtype=np.uint8)),
           "l.weight.absmax": rng.integers(0, 256, n // 64, dtype=np.uint8),
           "l.weight.quant_map": np.zeros(16, np.float32), "l.weight.nested_absmax": np.zeros(n // 64 // 256, np.float32),
           "l.weight.nested_quant_map": np.zeros(256, np.float32),
           "l.weight.quant_state.bitsandbytes__nf4": json_tensor({"quant_type": "nf4", "nested_dtype": "float32", "dtype": "bfloat16",
                                                                  "blocksize": 128, "nested_blocksize": 256, "nested_offset": 0.0,
                                                                  "shape": [OUT, IN]})}
    _refused(tmp_path, nf4, "l", message="NF4")


def test_malformed_files_are_refused(tmp_path):
    good = str(tmp_path / "g.safetensors")
    write_safetensors(good, {"a": np.arange(6, dtype=np.float32).reshape(2, 3)})
    raw = open(good, "rb").read()
    cases = {"short": raw[:6], "header_overrun": struct.pack("<Q", 1 << 40) + raw[8:], "truncated_data": raw[:-8],
             "not_json": struct.pack("<Q", 8) + b"notjson!" + raw[-24:]}
    for name, blob in cases.items():
        p = str(tmp_path / (name + ".safetensors"))
        open(p, "wb").write(blob)
        h = C.c_void_p()
        assert sfq.lib.sfq_checkpoint_open(p.encode(), C.byref(h)) != 0, name
        assert not h.value
    h = C.c_void_p()
    assert sfq.lib.sfq_checkpoint_open(str(tmp_path / "missing.safetensors").encode(), C.byref(h)) != 0


@pytest.mark.skipif(oracle.ref is None or not hasattr(oracle.ref, "ref_st_open"), reason="compiled reference not present")
def test_same_answers_as_the_reference_reader_and_detectors(checkpoint_path):
    path, tensors = checkpoint_path
    ref = oracle.ref
    V, I = C.c_void_p, C.c_int
    ref.ref_st_open.argtypes = [C.c_char_p, C.POINTER(V)]
    ref.ref_st_close.argtypes = [V]
    ref.ref_st_find.argtypes = [V, C.c_char_p, C.POINTER(I), C.POINTER(I), C.POINTER(C.c_int64), C.POINTER(V), C.POINTER(C.c_size_t)]
    for fn in (ref.ref_st_is_packed_int8, ref.ref_st_is_nf4):
        fn.argtypes = [V, C.c_char_p, C.POINTER(I)]
    ref.ref_st_packed_state.argtypes = [V, C.c_char_p, C.POINTER(I), C.POINTER(I), C.POINTER(I)]
    ref.ref_st_nf4_state.argtypes = [V, C.c_char_p, C.POINTER(I), C.POINTER(I), C.POINTER(C.c_float)]
    h = V()
    assert ref.ref_st_open(path.encode(), C.byref(h)) == 0
    try:
        with Checkpoint(path) as ck:
            for name in tensors:
                dt, rank, nb, data = I(), I(), C.c_size_t(), V()
                shape = (C.c_int64 * 8)()
                assert ref.ref_st_find(h, name.encode(), C.byref(dt), C.byref(rank), shape, C.byref(data), C.byref(nb)) == 0
                mine_dtype, mine_shape, mine_raw = ck.tensor(name)
                assert sfq.checkpoint.DTYPE_NAMES.index(mine_dtype) == dt.value, name  # same enumerator order as DType
                assert mine_shape == [shape[i] for i in range(rank.value)] and len(mine_raw) == nb.value
                assert np.array_equal(mine_raw, host_bytes(data.value, nb.value)), name
            layers = {"blocks.0.attn.out_proj": sfq.W4A8, "blocks.0.mlp.fc2": sfq.W6A8, "blocks.1.attn.out_proj": sfq.NVFP4,
                      "blocks.2.attn.out_proj": sfq.NF4, "blocks.3.mlp.fc1": sfq.F8E4M3, "text.proj": sfq.I8}
            for layer, fmt in layers.items():
                w = ck.linear(layer, OUT, IN, host=True)
                packed, nf4 = I(), I()
                assert ref.ref_st_is_packed_int8(h, (layer + ".weight").encode(), C.byref(packed)) == 0
                assert ref.ref_st_is_nf4(h, (layer + ".weight").encode(), C.byref(nf4)) == 0
                assert bool(packed.value) == (fmt in (sfq.W4A8, sfq.W6A8)) and bool(nf4.value) == (fmt == sfq.NF4)
                if packed.value:
                    bits, group, rot = I(), I(), I()
                    assert ref.ref_st_packed_state(h, (layer + ".weight").encode(), C.byref(bits), C.byref(group), C.byref(rot)) == 0
                    assert (bits.value, group.value, rot.value) == (6 if fmt == sfq.W6A8 else 4, w.packed_group_size, w.convrot_group)
                if nf4.value:
                    block, nested, off = I(), I(), C.c_float()
                    assert ref.ref_st_nf4_state(h, (layer + ".weight").encode(), C.byref(block), C.byref(nested), C.byref(off)) == 0
                    assert (block.value, nested.value, off.value) == (w.nf4_block_size, w.nf4_nested_block_size, w.nf4_nested_offset)
    finally:
        ref.ref_st_close(h)
