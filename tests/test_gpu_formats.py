"""The remaining weight formats of the runner's dense arm: F8E4M3, NF4 (double-quantized), F16, F32,
and the AWQ activation pre-scale. Streaming kernels are bit-exact against the oracle and against the
reference's own kernels; the Linear on top of them is checked against the fp64 product of the
dequantized operands (the reference's tolerance for its dense arm, tests/test_nn_kernels_linear_synthetic.cu:609-709)
and against the reference's LinearRunner."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import bf16_tensor, bits, dev, gaussian_bf16, ref_check, ref_dev, ref_weight_from

pytestmark = pytest.mark.gpu
P = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731


def _f8_codes(rng, n):
    codes = rng.integers(0, 256, size=n, dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3C  # the two NaN encodings carry no agreed bf16 payload
    return codes


def _nf4_state(rng, n_elems, block, nested):
    """Storage-form NF4 state with a generic sorted 16-entry map in [-1, 1]."""
    quant_map = np.sort(np.concatenate([[-1.0, 0.0, 1.0], rng.uniform(-1, 1, 13)])).astype(np.float32)
    packed = rng.integers(0, 256, size=(n_elems + 1) // 2, dtype=np.uint8)
    blocks = (n_elems + block - 1) // block
    absmax = rng.integers(0, 256, size=blocks, dtype=np.uint8)
    nested_map = np.sort(rng.uniform(-1, 1, 256)).astype(np.float32)
    nested_absmax = rng.uniform(0.01, 0.08, size=(blocks + nested - 1) // nested).astype(np.float32)
    return packed, absmax, quant_map, nested_map, nested_absmax


@pytest.mark.parametrize("n", [1, 7, 8, 4099, 1 << 20])
def test_f8e4m3_unpack_bit_exact(n):
    rng = np.random.default_rng(n)
    codes = _f8_codes(rng, n)
    scale = np.array([0.0123], np.float32)
    want = np.empty(n, np.uint16)
    oracle.lib.orc_f8_dequant_bf16(P(codes), float(scale[0]), n, P(want))
    d_codes, d_scale = dev(codes), dev(scale)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    sfq.check(sfq.lib.sfq_unpack_f8e4m3_bf16(sfq.ptr(d_codes), sfq.ptr(d_scale), sfq.ptr(out), n, None))
    assert np.array_equal(bits(out), want)
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(out)
        ref_check(ref, ref.ref_dev_dequant_f8(sfq.ptr(d_codes), sfq.ptr(d_scale), sfq.ptr(r), n))
        assert np.array_equal(bits(r), want)


def test_f8e4m3_unpack_every_code():
    codes = np.arange(256, dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0
    scale = np.array([1.0], np.float32)
    d_codes, d_scale = dev(codes), dev(scale)
    out = torch.empty(256, dtype=torch.bfloat16, device="cuda")
    sfq.check(sfq.lib.sfq_unpack_f8e4m3_bf16(sfq.ptr(d_codes), sfq.ptr(d_scale), sfq.ptr(out), 256, None))
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).to(torch.float32)
    assert torch.equal(out.float().cpu(), want)  # every e4m3 value is exact in bf16


@pytest.mark.parametrize("out_f,in_f,block,nested", [(3, 64, 64, 256), (33, 192, 64, 4), (64, 1024, 128, 16), (5, 6, 2, 3)])
def test_nf4_unpack_bit_exact(out_f, in_f, block, nested):
    n = out_f * in_f
    rng = np.random.default_rng(n + block)
    packed, absmax, qmap, nmap, nabs = _nf4_state(rng, n, block, nested)
    offset = 0.031
    want = np.empty(n, np.uint16)
    oracle.lib.orc_nf4_dequant_bf16(P(packed), P(absmax), P(qmap), P(nmap), P(nabs), block, nested, offset, n, P(want))
    d = [dev(a) for a in (packed, absmax, qmap, nmap, nabs)]
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    sfq.check(sfq.lib.sfq_unpack_nf4_bf16(*[sfq.ptr(t) for t in d], block, nested, offset, sfq.ptr(out), out_f, in_f, None))
    assert np.array_equal(bits(out), want)
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(out)
        ref_check(ref, ref.ref_dev_dequant_nf4(*[sfq.ptr(t) for t in d], block, nested, offset, sfq.ptr(r), out_f, in_f))
        assert np.array_equal(bits(r), want)


@pytest.mark.parametrize("rows,dim", [(1, 1), (3, 257), (64, 5120)])
def test_pre_quant_scale_bit_exact(rows, dim):
    x = gaussian_bf16((rows, dim), seed=rows)
    s = oracle.to_bf16(np.random.default_rng(dim).uniform(0.25, 4.0, dim).astype(np.float32))
    want = np.empty((rows, dim), np.uint16)
    oracle.lib.orc_pre_quant_scale_bf16(P(x), P(s), rows, dim, P(want))
    dx, ds = bf16_tensor(x), bf16_tensor(s)
    out = torch.empty_like(dx)
    sfq.check(sfq.lib.sfq_pre_quant_scale(sfq.ptr(dx), sfq.ptr(ds), sfq.ptr(out), rows, dim, None))
    assert np.array_equal(bits(out), want)
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(dx)
        ref_check(ref, ref.ref_dev_pre_quant_scale(sfq.ptr(dx), sfq.ptr(ds), sfq.ptr(r), rows, dim))
        assert np.array_equal(bits(r), want)


def _check_linear(w, keep, xb, wdq_bits, pre_scale_bits=None, group=0, bias_bits=None):
    """Runner output against the fp64 product of what the kernels feed the GEMM, and against the reference runner."""
    M = xb.shape[0]
    x = bf16_tensor(xb)
    y = sfq.LinearRunner().forward(w, x)
    assert sfq.device_status() == 0
    xin = xb
    if pre_scale_bits is not None:
        t = np.empty_like(xin)
        oracle.lib.orc_pre_quant_scale_bf16(P(xin), P(pre_scale_bits), M, xin.shape[1], P(t))
        xin = t
    if group:
        xin = oracle.convrot_bf16(xin, group)
    want = oracle.from_bf16(xin).astype(np.float64) @ oracle.from_bf16(wdq_bits).astype(np.float64).T
    if bias_bits is not None:
        want = want + oracle.from_bf16(bias_bits)
    got = oracle.from_bf16(bits(y))
    assert np.all(np.abs(got - want) <= 2e-3 + 2e-2 * np.abs(want))
    ref = ref_dev()
    if ref is not None:
        rw = ref_weight_from(w)
        yr = torch.empty_like(y)
        ms = C.c_float(0)
        ref_check(ref, ref.ref_dev_linear_forward(C.byref(rw), sfq.ptr(x), M, sfq.ptr(yr), 0, 0, C.byref(ms)))
        theirs = oracle.from_bf16(bits(yr))
        # two bf16 GEMMs with different summation orders: agree to output rounding
        assert np.all(np.abs(got - theirs) <= 2e-3 + 2e-2 * np.abs(theirs))
    del keep


def test_f8e4m3_linear():
    M, N, K = 70, 256, 384
    rng = np.random.default_rng(50)
    codes = _f8_codes(rng, N * K).reshape(N, K)
    codes &= 0xBF  # keep |value| < 2 so the products stay in the tolerance's useful range
    scale = np.array([0.04], np.float32)
    wdq = np.empty((N, K), np.uint16)
    oracle.lib.orc_f8_dequant_bf16(P(codes), float(scale[0]), N * K, P(wdq))
    keep = [dev(codes), dev(scale)]
    w = sfq.new_weight(format=sfq.F8E4M3, data=sfq.ptr(keep[0]), out_features=N, in_features=K,
                       weight_scale=sfq.ptr(keep[1]))
    _check_linear(w, keep, gaussian_bf16((M, K), seed=51), wdq)


def test_nf4_linear_with_awq_pre_scale():
    M, N, K = 33, 128, 512
    rng = np.random.default_rng(60)
    packed, absmax, qmap, nmap, nabs = _nf4_state(rng, N * K, 64, 256)
    wdq = np.empty((N, K), np.uint16)
    oracle.lib.orc_nf4_dequant_bf16(P(packed), P(absmax), P(qmap), P(nmap), P(nabs), 64, 256, 0.02, N * K, P(wdq))
    pre = oracle.to_bf16(rng.uniform(0.5, 2.0, K).astype(np.float32))
    bias = oracle.to_bf16((0.01 * rng.standard_normal(N)).astype(np.float32))
    keep = [dev(a) for a in (packed, absmax, qmap, nmap, nabs)] + [bf16_tensor(pre), bf16_tensor(bias)]
    w = sfq.new_weight(format=sfq.NF4, data=sfq.ptr(keep[0]), out_features=N, in_features=K, nf4_absmax=sfq.ptr(keep[1]),
                       nf4_quant_map=sfq.ptr(keep[2]), nf4_nested_quant_map=sfq.ptr(keep[3]),
                       nf4_nested_absmax=sfq.ptr(keep[4]), nf4_block_size=64, nf4_nested_block_size=256,
                       nf4_nested_offset=0.02, pre_quant_scale=sfq.ptr(keep[5]), bias=sfq.ptr(keep[6]),
                       bias_format=sfq.BF16)
    _check_linear(w, keep, gaussian_bf16((M, K), seed=61), wdq, pre_scale_bits=pre, bias_bits=bias)


@pytest.mark.parametrize("fmt", ["f16", "f32"])
def test_wide_float_weight_linear(fmt):
    M, N, K = 40, 128, 320
    rng = np.random.default_rng(70)
    wf = (0.05 * rng.standard_normal((N, K))).astype(np.float32)
    if fmt == "f16":
        stored = wf.astype(np.float16)
        wdq = np.empty((N, K), np.uint16)
        oracle.lib.orc_f16_to_bf16_n(P(stored.view(np.uint16)), P(wdq), N * K)
        keep = [torch.from_numpy(stored).cuda()]
        code = sfq.F16
    else:
        wdq = oracle.to_bf16(wf)
        keep = [torch.from_numpy(wf).cuda()]
        code = sfq.F32
    w = sfq.new_weight(format=code, data=sfq.ptr(keep[0]), out_features=N, in_features=K)
    _check_linear(w, keep, gaussian_bf16((M, K), seed=71), wdq)


def test_nvfp4_dense_arm_with_awq_pre_scale_skips_native_gemm():
    # A layer with pre_quant_scale never takes the native fp4 GEMM (src/cuda/linear.cu:120-139); it runs
    # pre-scale -> dense bf16 GEMM on the dequantized weight.
    from helpers import pack_nvfp4
    M, N, K = 48, 256, 512
    rng = np.random.default_rng(80)
    wf = (0.03 * rng.standard_normal((N, K))).astype(np.float32)
    data, scale, g = pack_nvfp4(wf)
    wdq = oracle.nvfp4_dequant_bf16(data, scale, g, N, K)
    pre = oracle.to_bf16(rng.uniform(0.5, 2.0, K).astype(np.float32))
    keep = [dev(data), dev(scale), bf16_tensor(pre)]
    w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(keep[0]), out_features=N, in_features=K,
                       block_scale=sfq.ptr(keep[1]), global_scale=g, pre_quant_scale=sfq.ptr(keep[2]))
    _check_linear(w, keep, gaussian_bf16((M, K), seed=81), wdq, pre_scale_bits=pre)
