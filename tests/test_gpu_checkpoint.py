"""A layer loaded from a safetensors file gives the same bits as the same layer built from arrays in memory."""
import ctypes as C

import numpy as np
import pytest
import torch

import slopfab_b200 as sfq
from helpers import bf16_tensor, dev, gaussian_bf16, pack_nvfp4, synthetic_packed_int8
from slopfab_b200.checkpoint import Checkpoint, json_tensor, write_safetensors

pytestmark = pytest.mark.gpu


def test_layers_from_a_file_match_layers_from_memory(tmp_path):
    N, K, M = 768, 512, 130
    rng = np.random.default_rng(31)
    packed, s_rel, s_ch, book = synthetic_packed_int8(4, 16, N, K, seed=32)
    wf = (0.03 * rng.standard_normal((N, K))).astype(np.float32)
    data, scale, g = pack_nvfp4(wf)
    f8 = rng.integers(0, 0x70, (N, K), dtype=np.uint8)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {
        "blocks.0.attn.qkv_proj.weight": ("U8", [N, K // 2], packed.view(np.uint8)),
        "blocks.0.attn.qkv_proj.weight_s_rel": ("F8_E4M3", [N, K // 16], s_rel),
        "blocks.0.attn.qkv_proj.weight_s_channel": s_ch,
        "blocks.0.attn.qkv_proj.weight_codebook": book,
        "blocks.0.attn.qkv_proj.comfy_quant": json_tensor({"format": "asym_w4a8_int8", "group_size": 16, "convrot_groupsize": 256}),
        "blocks.1.attn.qkv_proj.weight": ("U8", [N, K // 2], data),
        "blocks.1.attn.qkv_proj.weight_scale": ("F8_E4M3", [N, K // 16], scale),
        "blocks.1.attn.qkv_proj.weight_scale_2": np.array([g], np.float32),
        "blocks.2.mlp.fc1.weight": ("F8_E4M3", [N, K], f8),
        "blocks.2.mlp.fc1.weight_scale": np.array([0.03], np.float32),
    })
    x = bf16_tensor(gaussian_bf16((M, K), seed=33, outliers=True))
    runner = sfq.LinearRunner()
    runner.set_native(True)
    with Checkpoint(path) as ck:
        # W4A8
        keep = [dev(packed), dev(s_rel), dev(s_ch), dev(book)]
        direct = sfq.new_weight(format=sfq.W4A8, data=sfq.ptr(keep[0]), out_features=N, in_features=K, block_scale=sfq.ptr(keep[1]),
                                weight_scale=sfq.ptr(keep[2]), w4_codebook=sfq.ptr(keep[3]), packed_group_size=16, convrot=1,
                                convrot_group=256)
        loaded = ck.linear("blocks.0.attn.qkv_proj", N, K)
        want = runner.forward(direct, x)
        assert torch.equal(runner.forward(loaded, x), want)
        # q / k / v as views over the loaded fused weight
        for i in range(3):
            view = sfq.QuantWeight()
            sfq.check(sfq.lib.sfq_weight_row_block(C.byref(loaded), 3, i, C.byref(view)))
            assert torch.equal(runner.forward(view, x), want[:, i * 256:(i + 1) * 256])
        # NVFP4 (native fp4 path)
        keep4 = [dev(data), dev(scale)]
        direct4 = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep4[0]), out_features=N, in_features=K,
                                 block_scale=sfq.ptr(keep4[1]), global_scale=g)
        loaded4 = ck.linear("blocks.1.attn.qkv_proj", N, K)
        assert loaded4.global_scale == np.float32(g)
        assert torch.equal(runner.forward(loaded4, x), runner.forward(direct4, x))
        # fp8 per tensor (dense arm)
        keep8 = [dev(f8), dev(np.array([0.03], np.float32))]
        direct8 = sfq.new_weight(format=sfq.F8E4M3, data=sfq.ptr(keep8[0]), out_features=N, in_features=K, weight_scale=sfq.ptr(keep8[1]))
        assert torch.equal(runner.forward(ck.linear("blocks.2.mlp.fc1", N, K), x), runner.forward(direct8, x))
        # asking twice hands out the same device buffers
        again = ck.linear("blocks.1.attn.qkv_proj", N, K)
        assert again.data == loaded4.data and again.block_scale == loaded4.block_scale
        assert sfq.device_status() == 0
