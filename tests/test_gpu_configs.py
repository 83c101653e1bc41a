"""The benchmark configurations at their FULL sizes, through the runner (C ABI).

Full-size outputs are checked through properties that do not need the whole CPU result: every output row of
the path depends on one input row only, so a random subset of rows is recomputed by the oracle and must match
(bit-exact for the integer formats, the stated tolerance for fp4); sharding the token axis must not change a
single bit; and the step must be deterministic.
"""
import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import bf16_tensor, bits, dev, gaussian_bf16, pack_nvfp4, pack_w4a8, pack_w6a8

pytestmark = pytest.mark.gpu


def _rows(M, count, seed):
    rng = np.random.default_rng(seed)
    picks = np.unique(np.concatenate([[0, 1, 127, 128, M - 1], rng.integers(0, M, size=count)]))
    return picks[picks < M]


def _int8_weight(fmt, packed, s_rel, s_ch, book, bias, group, n, k):
    keep = [dev(packed), dev(s_rel), dev(s_ch), dev(book) if book is not None else None, dev(bias) if bias is not None else None]
    w = sfq.new_weight(format=fmt, data=sfq.ptr(keep[0]), out_features=n, in_features=k, block_scale=sfq.ptr(keep[1]),
                       weight_scale=sfq.ptr(keep[2]), w4_codebook=sfq.ptr(keep[3]), packed_group_size=group, convrot=1,
                       convrot_group=256, bias=sfq.ptr(keep[4]))
    return w, keep


def test_config2_w4a8_attention_projection_full_size():
    # M=4096, K=N=5120, activations N(0,1) with 0.1 % outliers x20, fp32 bias, seed 1
    M, N, K = 4096, 5120, 5120
    rng = np.random.default_rng(1)
    packed, s_rel, s_ch, book = pack_w4a8((0.02 * rng.standard_normal((N, K))).astype(np.float32))
    bias = (0.01 * rng.standard_normal(N)).astype(np.float32)
    x = gaussian_bf16((M, K), seed=1, outliers=True)
    w, keep = _int8_weight(sfq.W4A8, packed, s_rel, s_ch, book, bias, 16, N, K)
    runner = sfq.LinearRunner()
    dx = bf16_tensor(x)
    y = runner.forward(w, dx)
    assert sfq.device_status() == 0
    picks = _rows(M, 48, seed=2)
    want = oracle.packed_int8_linear(np.ascontiguousarray(x[picks]), packed.view(np.uint8), s_rel, s_ch, book, 4, 16, N, K, bias=bias)
    got = bits(y)[picks]
    assert np.array_equal(got, want), f"{int((got != want).sum())} of {want.size} sampled outputs differ"
    # token sharding changes nothing: 8 ragged shards (as an 8-GPU run would own them) reproduce y bit for bit
    from slopfab_b200.parallel import token_shard
    y2 = torch.empty_like(y)
    for r in range(8):
        r0, rc = token_shard(M - 3, 8, r)  # ragged on purpose
        runner.forward(w, dx[r0:r0 + rc], y2[r0:r0 + rc])
    assert torch.equal(y[:M - 3].view(torch.int16), y2[:M - 3].view(torch.int16))
    # deterministic
    assert torch.equal(runner.forward(w, dx).view(torch.int16), y.view(torch.int16))


def test_config3_w6a8_ffn_pair_full_size():
    # up: M=32760, K=5120 -> N=13824 with GELU-tanh fused; down: 13824 -> 5120; W6A8 group 32; seed 2
    M, H, F = 32760, 5120, 13824
    rng = np.random.default_rng(2)
    up = pack_w6a8((0.02 * rng.standard_normal((F, H))).astype(np.float32), 32)
    down = pack_w6a8((0.02 * rng.standard_normal((H, F))).astype(np.float32), 32)
    x = gaussian_bf16((M, H), seed=2)
    w_up, k1 = _int8_weight(sfq.W6A8, up[0], up[1], up[2], None, None, 32, F, H)
    w_down, k2 = _int8_weight(sfq.W6A8, down[0], down[1], down[2], None, None, 32, H, F)
    runner = sfq.LinearRunner()
    dx = bf16_tensor(x)
    runner.set_activation(sfq.ACT_GELU_TANH)
    h = runner.forward(w_up, dx)
    runner.set_activation(sfq.ACT_NONE)
    y = runner.forward(w_down, h)
    assert sfq.device_status() == 0
    picks = _rows(M, 24, seed=3)
    # up-projection before the activation is bit-exact; the fused GELU is within one bf16 ulp of the host tanh
    pre = oracle.packed_int8_linear(np.ascontiguousarray(x[picks]), up[0].view(np.uint8), up[1], up[2], None, 6, 32, F, H)
    act = pre.copy()
    oracle.lib.orc_gelu_tanh_bf16(act.ctypes.data, act.size)
    got_h = bits(h)[picks]
    assert np.abs(got_h.astype(np.int32) - act.astype(np.int32)).max() <= 1
    # down-projection fed with the DEVICE's own hidden rows is bit-exact against the integer oracle
    want_y = oracle.packed_int8_linear(np.ascontiguousarray(got_h), down[0].view(np.uint8), down[1], down[2], None, 6, 32, H, F)
    got_y = bits(y)[picks]
    assert np.array_equal(got_y, want_y), f"{int((got_y != want_y).sum())} of {want_y.size} sampled outputs differ"
    assert np.isfinite(oracle.from_bf16(got_y)).all()


def test_config4_linears_nvfp4_full_token_count():
    # the four Linears of one block at 75600 tokens (21x45x80), hidden 5120, FFN 13824, NVFP4 native, seed 3
    M, H, F = 75600, 5120, 13824
    rng = np.random.default_rng(3)
    x = gaussian_bf16((M, H), seed=3)
    dx = bf16_tensor(x)
    runner = sfq.LinearRunner()
    runner.set_native(True)
    picks = _rows(M, 12, seed=4)
    xf = None
    for name, n, k in (("out", H, H), ("fc1", F, H), ("qkv", 3 * H, H), ("fc2", H, F)):
        if k == F and xf is None:  # fc2 reads an FFN-wide activation
            del dx
            torch.cuda.empty_cache()
            xf = gaussian_bf16((M, F), seed=5)
            x, dx = xf, bf16_tensor(xf)
        data, scale, g = pack_nvfp4((0.02 * rng.standard_normal((n, k))).astype(np.float32))
        keep = [dev(data), dev(scale)]
        w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep[0]), out_features=n, in_features=k,
                           block_scale=sfq.ptr(keep[1]), global_scale=g)
        y = runner.forward(w, dx)
        assert sfq.device_status() == 0
        want = oracle.nvfp4_linear(np.ascontiguousarray(x[picks]), data, scale, g, n, k)
        max_abs, rel_l2, corr = oracle.compare_bf16(want, bits(y)[picks])
        assert max_abs <= 2e-2 and rel_l2 <= 1e-3, (name, max_abs, rel_l2, corr)
        del y
        torch.cuda.empty_cache()


@pytest.mark.parametrize("kind", ["nvfp4", "w4a8"])
@pytest.mark.parametrize("name,k,n", [("attn_proj", 5120, 5120), ("ffn_up", 5120, 13824), ("ffn_down", 13824, 5120)])
def test_config5_linears_at_one_gpus_share_of_the_tokens(kind, name, k, n):
    # the scaling sweep's Linears at the rows one of eight GPUs owns: 111600 / 8 = 13950 (not a multiple of any tile
    # height), distributions of configs 1-2 (activations N(0,1) with 0.1 % outliers x20, weights N(0,0.02)), seed 4
    from slopfab_b200.parallel import token_shard
    M = token_shard(31 * 45 * 80, 8, 3)[1]
    assert M == 13950
    rng = np.random.default_rng(4)
    wf = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    x = gaussian_bf16((M, k), seed=4, outliers=True)
    dx = bf16_tensor(x)
    picks = _rows(M, 16, seed=5)
    runner = sfq.LinearRunner()
    if kind == "nvfp4":
        data, scale, g = pack_nvfp4(wf)
        keep = [dev(data), dev(scale)]
        w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep[0]), out_features=n, in_features=k, block_scale=sfq.ptr(keep[1]),
                           global_scale=g)
        runner.set_native(True)
        y = runner.forward(w, dx)
        assert sfq.device_status() == 0
        want = oracle.nvfp4_linear(np.ascontiguousarray(x[picks]), data, scale, g, n, k)
        max_abs, rel_l2, corr = oracle.compare_bf16(want, bits(y)[picks])
        assert max_abs <= 2e-2 and rel_l2 <= 1e-3, (name, max_abs, rel_l2, corr)
    else:
        packed, s_rel, s_ch, book = pack_w4a8(wf)
        w, keep = _int8_weight(sfq.W4A8, packed, s_rel, s_ch, book, None, 16, n, k)
        y = runner.forward(w, dx)
        assert sfq.device_status() == 0
        want = oracle.packed_int8_linear(np.ascontiguousarray(x[picks]), packed.view(np.uint8), s_rel, s_ch, book, 4, 16, n, k)
        got = bits(y)[picks]
        assert np.array_equal(got, want), f"{name}: {int((got != want).sum())} of {want.size} sampled outputs differ"
    # the last, partial row tile holds real rows only: nothing past row M - 1 was written
    assert torch.isfinite(y.float()).all()
