"""GPU parity of the LinearRunner through the C ABI: the reference's end-to-end known-answer tests for
W4A8 / W6A8 (bit-exact bf16), prepare + forward_prepared == forward, the NVFP4 arms, and the error contract."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import (bf16_tensor, bits, dev, gaussian_bf16, pack_nvfp4, pack_w4a8, pack_w6a8, ref_check, ref_dev,
                     ref_weight_from, synthetic_packed_int8)
from test_oracle_golden import _packed_case

pytestmark = pytest.mark.gpu


def _packed_weight(bits_, group, n, k, packed, s_rel, s_ch, book, bias=None, bias_format=sfq.F32):
    keep = [dev(packed), dev(s_rel), dev(s_ch)] + ([dev(book)] if bits_ == 4 else []) + ([bias] if bias is not None else [])
    w = sfq.new_weight(format=sfq.W4A8 if bits_ == 4 else sfq.W6A8, data=sfq.ptr(keep[0]), out_features=n,
                       in_features=k, block_scale=sfq.ptr(keep[1]), weight_scale=sfq.ptr(keep[2]),
                       packed_group_size=group, w4_codebook=sfq.ptr(keep[3]) if bits_ == 4 else None, convrot=1,
                       convrot_group=256, bias=sfq.ptr(bias) if bias is not None else None, bias_format=bias_format)
    return w, keep


@pytest.mark.parametrize("bits_,group", [(4, 16), (6, 16), (6, 32), (6, 64)])
def test_packed_integer_linear_known_answer(bits_, group):
    # nn_w4a8_native_bf16_linear / nn_w6a8_native_bf16_linear (tests/test_nn_kernels_linear_synthetic.cu:820-890)
    packed, levels, scales, book, channel, x = _packed_case(bits_, group)
    w, keep = _packed_weight(bits_, group, 4, 256, packed.view(np.int8), scales, channel, book)
    runner = sfq.LinearRunner()
    xb = oracle.to_bf16(x)
    y = runner.forward(w, bf16_tensor(xb))
    want = oracle.packed_int8_linear(xb, packed, scales, channel, book if bits_ == 4 else None, bits_, group, 4, 256)
    assert np.array_equal(bits(y), want)
    runner.set_native(True)  # must change nothing
    assert np.array_equal(bits(runner.forward(w, bf16_tensor(xb))), want)
    assert sfq.device_status() == 0


@pytest.mark.parametrize("bits_,group,M,N,K", [(4, 16, 333, 640, 1024), (6, 32, 130, 384, 2560), (4, 16, 4100, 2048, 256)])
def test_packed_integer_linear_against_oracle_and_reference(bits_, group, M, N, K):
    packed, s_rel, s_ch, book = synthetic_packed_int8(bits_, group, N, K, seed=M)
    rng = np.random.default_rng(M)
    bias = (0.01 * rng.standard_normal(N)).astype(np.float32)
    dbias = dev(bias)
    w, keep = _packed_weight(bits_, group, N, K, packed, s_rel, s_ch, book, bias=dbias)
    xb = gaussian_bf16((M, K), seed=N, outliers=True)
    dx = bf16_tensor(xb)
    runner = sfq.LinearRunner()
    y = runner.forward(w, dx)
    assert sfq.device_status() == 0
    want, inter = oracle.packed_int8_linear(xb, packed.view(np.uint8), s_rel, s_ch, book, bits_, group, N, K, bias=bias,
                                            want_intermediates=True)
    bad = int((bits(y) != want).sum())
    assert bad == 0, f"{bad} of {M * N} bf16 outputs differ from the integer oracle"
    ref = ref_dev()
    if ref is not None:
        # the reference's own LinearRunner on the same device buffers: identical bf16 bits, identical accumulators
        rw = ref_weight_from(w)
        y2 = torch.empty_like(y)
        ref_check(ref, ref.ref_dev_linear_forward(C.byref(rw), sfq.ptr(dx), M, sfq.ptr(y2), 0, 0, None))
        assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
        codes = torch.empty((N, K), dtype=torch.int8, device="cuda")
        rot = torch.empty((M, K), dtype=torch.bfloat16, device="cuda")
        act = torch.empty((M, K), dtype=torch.int8, device="cuda")
        sc = torch.empty(M, dtype=torch.float32, device="cuda")
        acc = torch.empty((M, N), dtype=torch.int32, device="cuda")
        ref_check(ref, ref.ref_dev_packed_int8_accumulate(C.byref(rw), sfq.ptr(dx), M, sfq.ptr(codes), sfq.ptr(rot),
                                                          sfq.ptr(act), sfq.ptr(sc), sfq.ptr(acc)))
        assert np.array_equal(acc.cpu().numpy(), inter["acc"])
        assert np.array_equal(act.cpu().numpy(), inter["q"]) and np.array_equal(codes.cpu().numpy(), inter["w8"])
    # GELU fused into the epilogue == the reference's separate launch on the bf16 result
    runner.set_activation(sfq.ACT_GELU_TANH)
    yg = runner.forward(w, dx)
    if ref is not None:
        ref_check(ref, ref.ref_dev_gelu_tanh(sfq.ptr(y), y.numel()))
        assert torch.equal(yg.view(torch.int16), y.view(torch.int16))


def test_prepare_then_chunks_is_bit_identical_to_forward():
    # linear_prepared_matches_per_chunk (tests/test_nn_kernels_linear_synthetic.cu:511-607)
    M, N, K, chunk = 700, 512, 1024, 256
    for fmt in ("w4a8", "nvfp4_native", "nvfp4_dequant"):
        xb = gaussian_bf16((M, K), seed=11)
        dx = bf16_tensor(xb)
        runner = sfq.LinearRunner()
        if fmt == "w4a8":
            packed, s_rel, s_ch, book = synthetic_packed_int8(4, 16, N, K, seed=2)
            w, keep = _packed_weight(4, 16, N, K, packed, s_rel, s_ch, book)
        else:
            rng = np.random.default_rng(4)
            data, scale, g = pack_nvfp4((0.02 * rng.standard_normal((N, K))).astype(np.float32))
            keep = [dev(data), dev(scale)]
            w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep[0]), out_features=N, in_features=K,
                               block_scale=sfq.ptr(keep[1]), global_scale=g)
            runner.set_native(fmt == "nvfp4_native")
        whole = runner.forward(w, dx).clone()
        prepared, used = runner.prepare(w, chunk)
        assert (prepared is None) == (fmt == "nvfp4_native")
        y = torch.empty_like(whole)
        for r0 in range(0, M, chunk):
            r1 = min(M, r0 + chunk)
            runner.forward_prepared(w, prepared, used, dx[r0:r1], y[r0:r1])
        assert torch.equal(whole.view(torch.int16), y.view(torch.int16)), fmt
        assert sfq.device_status() == 0


def test_nvfp4_linear_both_semantics():
    # linear_nvfp4 (tests/test_nn_kernels_nvfp4_synthetic.cu:130-237): native off = dequantize + bf16 GEMM
    # against cpu_matmul_nt(x, dequantized W); native on = fp4 activations against the fp4-activation reference.
    M, N, K = 200, 256, 320
    rng = np.random.default_rng(21)
    wf = (0.02 * rng.standard_normal((N, K))).astype(np.float32)
    bias = (0.01 * rng.standard_normal(N)).astype(np.float32)
    data, scale, g = pack_nvfp4(wf)
    xb = gaussian_bf16((M, K), seed=22)
    keep = [dev(data), dev(scale), dev(bias)]
    w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep[0]), out_features=N, in_features=K,
                       block_scale=sfq.ptr(keep[1]), global_scale=g, bias=sfq.ptr(keep[2]))
    runner = sfq.LinearRunner()
    y0 = runner.forward(w, bf16_tensor(xb))
    want0 = oracle.from_bf16(oracle.nvfp4_linear_dequant(xb, data, scale, g, N, K, bias=bias))
    got0 = oracle.from_bf16(bits(y0))
    assert np.all(np.abs(got0 - want0) <= 1e-3 + 1e-2 * np.abs(want0))
    ref = ref_dev()
    if ref is not None:  # the reference's dequantize + cuBLAS result for the same bytes
        y2 = torch.empty_like(y0)
        rw = ref_weight_from(w)
        dxr = bf16_tensor(xb)
        ref_check(ref, ref.ref_dev_linear_forward(C.byref(rw), sfq.ptr(dxr), M, sfq.ptr(y2), 0, 0, None))
        r = oracle.from_bf16(bits(y2))
        assert np.all(np.abs(got0 - r) <= 1e-3 + 1e-2 * np.abs(r))
    runner.set_native(True)
    y1 = runner.forward(w, bf16_tensor(xb))
    want1 = oracle.nvfp4_linear(xb, data, scale, g, N, K, bias=bias)
    max_abs, rel_l2, corr = oracle.compare_bf16(want1, bits(y1))
    assert max_abs <= 2e-2 and rel_l2 <= 1e-3, (max_abs, rel_l2)
    assert sfq.device_status() == 0


def test_runner_error_contract():
    runner = sfq.LinearRunner()
    packed, s_rel, s_ch, book = synthetic_packed_int8(4, 16, 128, 256, seed=1)
    w, keep = _packed_weight(4, 16, 128, 256, packed, s_rel, s_ch, book)
    x = bf16_tensor(gaussian_bf16((4, 256), seed=1))
    y = torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda")
    # rows <= 0 is a silent no-op (src/cuda/linear.cu:153-154)
    sfq.check(sfq.lib.sfq_linear_forward(runner._h, C.byref(w), sfq.ptr(x), 0, sfq.ptr(y), None, 0))
    assert not y.any()
    # each violated precondition of src/cuda/linear.cu:179-187 is std::invalid_argument
    for field, value in (("convrot", 0), ("convrot_group", 64), ("block_scale", None), ("weight_scale", None),
                         ("w4_codebook", None), ("packed_group_size", 32), ("full_precision", 1)):
        bad = sfq.new_weight(**{n: getattr(w, n) for n, _ in sfq.QuantWeight._fields_})
        setattr(bad, field, value)
        with pytest.raises(sfq.SfqError) as e:
            runner.forward(bad, x)
        assert e.value.code == sfq.ERR_INVALID_ARGUMENT, field
    w6 = sfq.new_weight(**{n: getattr(w, n) for n, _ in sfq.QuantWeight._fields_})
    w6.format = sfq.W6A8  # W6 with a codebook is refused
    with pytest.raises(sfq.SfqError):
        runner.forward(w6, x)
    # a dense-form weight with a null prepared pointer throws rather than running the wrong GEMM
    wb = sfq.new_weight(format=sfq.BF16, data=sfq.ptr(x), out_features=4, in_features=256)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    rc = sfq.lib.sfq_linear_forward_prepared(runner._h, C.byref(wb), None, sfq.ptr(x), 4, sfq.ptr(y), sfq.ptr(ws), ws.numel())
    assert rc == sfq.ERR_RUNTIME and b"prepare" in sfq.lib.sfq_last_error()
    # an arena that is too small is reported, not overrun
    rc = sfq.lib.sfq_linear_forward(runner._h, C.byref(w), sfq.ptr(x), 4, sfq.ptr(y), sfq.ptr(ws), 1024)
    assert rc == sfq.ERR_OUT_OF_MEMORY
    # an fp8 weight without its scale is refused (materialise_bf16, src/cuda/linear_weights.cu:580-634)
    wf8 = sfq.new_weight(format=sfq.F8E4M3, data=sfq.ptr(x), out_features=4, in_features=256)
    with pytest.raises(sfq.SfqError):
        runner.forward(wf8, x)


@pytest.mark.parametrize("group", [256, 64, 0])
def test_int8_weight_only_arm(group):
    # linear_int8_convrot (tests/test_nn_kernels_linear_synthetic.cu:609-709): INT8 per-channel weight, online
    # ConvRot of the activation, dequantize + bf16 GEMM; 2e-3 abs / 2e-2 rel against the fp64 product.
    import ctypes as C
    M, N, K = 70, 256, 512
    rng = np.random.default_rng(31 + group)
    wf = (0.05 * rng.standard_normal((N, K))).astype(np.float32)
    codes = np.zeros((N, K), np.int8)
    scale = np.zeros(N, np.float32)
    P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    sfq.check(sfq.lib.sfq_pack_int8(P(wf), N, K, group, P(codes), P(scale)))
    bias = oracle.to_bf16((0.01 * rng.standard_normal(N)).astype(np.float32))
    xb = gaussian_bf16((M, K), seed=32)
    keep = [dev(codes), dev(scale), bf16_tensor(bias)]
    w = sfq.new_weight(format=sfq.I8, data=sfq.ptr(keep[0]), out_features=N, in_features=K, weight_scale=sfq.ptr(keep[1]),
                       per_channel_scale=1, convrot=1 if group else 0, convrot_group=group or 256, bias=sfq.ptr(keep[2]),
                       bias_format=sfq.BF16)
    y = sfq.LinearRunner().forward(w, bf16_tensor(xb))
    assert sfq.device_status() == 0
    wdq = np.empty((N, K), np.uint16)
    oracle.lib.orc_int8_dequant_bf16(P(codes), P(scale), N, K, P(wdq))
    xr = oracle.convrot_bf16(xb, group) if group else xb
    want = oracle.from_bf16(xr).astype(np.float64) @ oracle.from_bf16(wdq).astype(np.float64).T + oracle.from_bf16(bias)
    got = oracle.from_bf16(bits(y))
    assert np.all(np.abs(got - want) <= 2e-3 + 2e-2 * np.abs(want))
    # and it really is the rotated product: without rotating x the result is far away (x H W^T is noise)
    if group:
        wrong = oracle.from_bf16(xb).astype(np.float64) @ oracle.from_bf16(wdq).astype(np.float64).T
        assert np.sqrt(((got - wrong) ** 2).sum() / (wrong ** 2).sum()) > 0.5


def test_bf16_weight_arm():
    M, N, K = 65, 384, 520
    x = gaussian_bf16((M, K), seed=40)
    wb = gaussian_bf16((N, K), seed=41, sigma=0.05)
    keep = [bf16_tensor(wb)]
    w = sfq.new_weight(format=sfq.BF16, data=sfq.ptr(keep[0]), out_features=N, in_features=K)
    y = sfq.LinearRunner().forward(w, bf16_tensor(x))
    want = oracle.from_bf16(x).astype(np.float64) @ oracle.from_bf16(wb).astype(np.float64).T
    got = oracle.from_bf16(bits(y))
    assert np.all(np.abs(got - want) <= 1e-3 + 1e-2 * np.abs(want))


def test_runner_swiglu_activation_matches_gemm_then_swiglu():
    # the H3 block's mlp.fc1 is [gate | up] followed by launch_swiglu (src/dit/transformer_execution.cpp); with
    # set_activation(ACT_SWIGLU) the runner writes silu(gate) * up directly, same bits
    M, N, K = 300, 1024, 512
    packed, s_rel, s_ch, book = synthetic_packed_int8(4, 16, N, K, seed=11)
    w, keep = _packed_weight(4, 16, N, K, packed, s_rel, s_ch, book)
    x = bf16_tensor(gaussian_bf16((M, K), seed=12, outliers=True))
    plain = sfq.LinearRunner().forward(w, x)
    want = torch.empty((M, N // 2), dtype=torch.bfloat16, device="cuda")
    sfq.check(sfq.lib.sfq_swiglu(sfq.ptr(plain), sfq.ptr(want), M, N // 2, None))
    runner = sfq.LinearRunner()
    runner.set_activation(sfq.ACT_SWIGLU)
    got = runner.forward(w, x)
    assert got.shape == (M, N // 2)
    assert sfq.device_status() == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("fmt", ["nvfp4", "w4a8"])
def test_qkv_views_over_a_fused_weight(fmt):
    # three views from sfq_weight_row_block give exactly the column blocks of the fused projection
    inner, K, M = 256, 512, 100
    x = bf16_tensor(gaussian_bf16((M, K), seed=21, outliers=True))
    if fmt == "nvfp4":
        wf = (0.03 * np.random.default_rng(22).standard_normal((3 * inner, K))).astype(np.float32)
        data, scale, g = pack_nvfp4(wf)
        keep = [dev(data), dev(scale)]
        fused = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep[0]), out_features=3 * inner, in_features=K,
                               block_scale=sfq.ptr(keep[1]), global_scale=g)
    else:
        packed, s_rel, s_ch, book = synthetic_packed_int8(4, 16, 3 * inner, K, seed=23)
        fused, keep = _packed_weight(4, 16, 3 * inner, K, packed, s_rel, s_ch, book)
    runner = sfq.LinearRunner()
    runner.set_native(True)
    whole = runner.forward(fused, x)
    for i in range(3):
        view = sfq.QuantWeight()
        sfq.check(sfq.lib.sfq_weight_row_block(C.byref(fused), 3, i, C.byref(view)))
        part = runner.forward(view, x)
        assert torch.equal(part.view(torch.int16), whole[:, i * inner:(i + 1) * inner].contiguous().view(torch.int16)), i
    assert sfq.device_status() == 0
