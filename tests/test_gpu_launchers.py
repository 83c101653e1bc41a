"""The small launchers of the reference's linear headers that sit beside the runner (fp32 ConvRot, int32 -> bf16 / fp32
output scaling, fp8 activation quantizer, NF4 -> fp16, the reference-layout fp4 GEMM entry, and the fp32-compute arm
with its ConvRot / AWQ front stages): each against a numpy statement of its arithmetic and, where the compiled
reference is present, bit for bit against the reference's own kernel on the same device buffers."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import P, bf16_tensor, bits, dev, gaussian_bf16, pack_nvfp4, ref_check, ref_dev, ref_weight_from
from test_gpu_formats import _nf4_state

pytestmark = pytest.mark.gpu

H4 = np.array([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], np.float64)


def _kron_power(stages):
    h = np.ones((1, 1))
    for _ in range(stages):
        h = np.kron(H4, h)  # stride 1 is the innermost base-4 digit
    return h


@pytest.mark.parametrize("rows,dim,group", [(5, 1280, 256), (3, 768, 256), (7, 64, 16), (2, 12, 4), (1, 2048, 1024)])
def test_convrot_f32(rows, dim, group):
    rng = np.random.default_rng(rows * dim)
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    dx = dev(x)
    out = torch.empty_like(dx)
    sfq.check(sfq.lib.sfq_convrot_f32(sfq.ptr(dx), sfq.ptr(out), rows, dim, group, None))
    stages = {4: 1, 16: 2, 64: 3, 256: 4, 1024: 5}[group]
    h = _kron_power(stages) / np.sqrt(group)
    want = (x.reshape(rows, dim // group, group).astype(np.float64) @ h.T).reshape(rows, dim)
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-5  # the reference's own bound for this transform
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(dx)
        ref_check(ref, ref.ref_dev_convrot_f32(sfq.ptr(dx), sfq.ptr(r), rows, dim, group))
        assert torch.equal(r.view(torch.int32), out.view(torch.int32))
    with pytest.raises(sfq.SfqError, match="power of four"):
        sfq.check(sfq.lib.sfq_convrot_f32(sfq.ptr(dx), sfq.ptr(out), rows, dim, 8 if dim % 8 == 0 else 2, None))


@pytest.mark.parametrize("rows,cols", [(3, 4), (37, 1000), (256, 5120)])
def test_int8_output_scaling(rows, cols):
    rng = np.random.default_rng(rows + cols)
    acc = rng.integers(-(1 << 24), 1 << 24, size=(rows, cols), dtype=np.int32)
    rs = (rng.random(rows) * 0.05 + 1e-3).astype(np.float32)
    cs = (rng.random(cols) * 0.01 + 1e-4).astype(np.float32)
    d_acc, d_rs, d_cs = dev(acc), dev(rs), dev(cs)
    y = torch.empty((rows, cols), dtype=torch.bfloat16, device="cuda")
    sfq.check(sfq.lib.sfq_int8_output_bf16(sfq.ptr(d_acc), sfq.ptr(d_rs), sfq.ptr(d_cs), sfq.ptr(y), rows, cols, None))
    f = (acc.astype(np.float32) * rs[:, None]) * cs[None, :]  # two fp32 roundings in this order
    assert np.array_equal(bits(y), oracle.to_bf16(f))
    io = d_acc.clone()
    sfq.check(sfq.lib.sfq_int8_output_f32(sfq.ptr(io), sfq.ptr(d_rs), sfq.ptr(d_cs), rows, cols, None))
    assert np.array_equal(io.view(torch.float32).cpu().numpy().view(np.uint32), f.view(np.uint32))
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(y)
        ref_check(ref, ref.ref_dev_output_bf16(sfq.ptr(d_acc), sfq.ptr(d_rs), sfq.ptr(d_cs), sfq.ptr(r), rows, cols))
        assert torch.equal(r.view(torch.int16), y.view(torch.int16))
        io2 = d_acc.clone()
        ref_check(ref, ref.ref_dev_output_f32(sfq.ptr(io2), sfq.ptr(d_rs), sfq.ptr(d_cs), rows, cols))
        assert torch.equal(io2, io)


def test_quantize_f8e4m3():
    x = gaussian_bf16((1, 70001), seed=8, sigma=3.0, outliers=True).reshape(-1)
    x[:6] = oracle.to_bf16(np.array([0.0, -0.0, 448.0, 1e6, -1e6, 2.0 ** -10], np.float32))
    dx = bf16_tensor(x)
    out = torch.empty(x.size, dtype=torch.uint8, device="cuda")
    sfq.check(sfq.lib.sfq_quantize_f8e4m3(sfq.ptr(dx), 0.037, sfq.ptr(out), x.size, None))
    scaled = torch.from_numpy(oracle.from_bf16(x) * np.float32(1.0 / np.float32(0.037)))
    want = scaled.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(out.cpu(), want)
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(out)
        ref_check(ref, ref.ref_dev_quantize_f8(sfq.ptr(dx), 0.037, sfq.ptr(r), x.size))
        assert torch.equal(r, out)
    with pytest.raises(sfq.SfqError, match="input_scale is zero"):
        sfq.check(sfq.lib.sfq_quantize_f8e4m3(sfq.ptr(dx), 0.0, sfq.ptr(out), x.size, None))


@pytest.mark.parametrize("n,block,nested", [(64 * 3, 64, 256), (4096 * 8, 64, 256), (33 * 192 + 1, 64, 4), (30, 2, 3)])
def test_nf4_to_f16(n, block, nested):
    rng = np.random.default_rng(n)
    packed, absmax, qmap, nmap, nabs = _nf4_state(rng, n, block, nested)
    d = [dev(a) for a in (packed, absmax, qmap, nmap, nabs)]
    out = torch.empty(n, dtype=torch.float16, device="cuda")
    sfq.check(sfq.lib.sfq_unpack_nf4_f16(*[sfq.ptr(t) for t in d], block, nested, 0.031, sfq.ptr(out), n, None))
    # the same decode the bf16 form is pinned to, narrowed to fp16 instead: value = map[code] * fma(nested, absmax2, offset)
    idx = np.arange(n)
    b = idx // block
    scale = (nmap[absmax[b]].astype(np.float64) * nabs[b // nested].astype(np.float64) + np.float64(np.float32(0.031))).astype(np.float32)
    codes = np.where(idx % 2 == 0, packed[idx // 2] >> 4, packed[idx // 2] & 15)
    want = (qmap[codes] * scale).astype(np.float16)
    # the scale here went through float64 (one more rounding than the kernel's fused multiply-add): allow one fp16 ulp
    got = out.cpu().numpy()
    assert np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32)).max() <= 1
    ref = ref_dev()
    if ref is not None:
        r = torch.empty_like(out)
        ref_check(ref, ref.ref_dev_dequant_nf4_f16(*[sfq.ptr(t) for t in d], block, nested, 0.031, sfq.ptr(r), n))
        assert torch.equal(r.view(torch.int16), out.view(torch.int16))


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (129, 256, 64), (200, 128, 320), (1000, 384, 1024)])
def test_nvfp4_gemm_from_reference_layout_activations(M, N, K):
    """nvfp4_gemm_forward_q's operand convention: activations quantized into the reference's layout give the same bits
    as the same activations quantized straight into the GEMM's own layout."""
    rng = np.random.default_rng(M + N + K)
    data, scale, g = pack_nvfp4((0.02 * rng.standard_normal((N, K))).astype(np.float32))
    dd, ds = dev(data), dev(scale)
    x = bf16_tensor(gaussian_bf16((M, K), seed=M))
    xq = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda")
    xs = torch.empty(M * K // 16, dtype=torch.uint8, device="cuda")
    sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(x), None, sfq.ptr(xq), sfq.ptr(xs), None, M, K, sfq.NVFP4_ACT_REFERENCE, None))
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    sfq.check(sfq.lib.sfq_gemm_nvfp4_reference_layout(sfq.ptr(xq), sfq.ptr(xs), sfq.ptr(dd), sfq.ptr(ds), g, sfq.ptr(got), M, N, K, None))
    fq = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda")
    fs = torch.empty(sfq.lib.sfq_nvfp4_act_scale_bytes(M, K), dtype=torch.uint8, device="cuda")
    sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(x), None, sfq.ptr(fq), sfq.ptr(fs), None, M, K, sfq.NVFP4_ACT_GEMM_FEED, None))
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    ep = sfq.Epilogue(None, None, g, None, sfq.F32, sfq.ACT_NONE)
    sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(fq), sfq.ptr(fs), sfq.ptr(dd), sfq.ptr(ds), C.byref(ep), sfq.ptr(want), M, N, K, None))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert sfq.device_status() == 0
    # and it is the fp4-activation arithmetic of the oracle
    ref_bits = oracle.nvfp4_linear(bits(x), data, scale, g, N, K)
    max_abs, rel_l2, _ = oracle.compare_bf16(ref_bits, bits(got))
    assert max_abs <= 2e-2 and rel_l2 <= 1e-3
    with pytest.raises(sfq.SfqError, match="out % 128"):
        sfq.check(sfq.lib.sfq_gemm_nvfp4_reference_layout(sfq.ptr(xq), sfq.ptr(xs), sfq.ptr(dd), sfq.ptr(ds), g, sfq.ptr(got), M, 100, K, None))


@pytest.mark.parametrize("fmt,convrot,awq", [("f32", True, False), ("bf16", True, True), ("f32", False, True)])
def test_forward_f32_with_convrot_and_awq_front_stages(fmt, convrot, awq):
    rows, n, k = 5, 192, 512
    rng = np.random.default_rng(n + k + convrot + 2 * awq)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = (0.05 * rng.standard_normal((n, k))).astype(np.float32)
    keep = []
    if fmt == "bf16":
        wb = oracle.to_bf16(w)
        w = oracle.from_bf16(wb)
        keep.append(dev(wb))
        weight = sfq.new_weight(format=sfq.BF16, data=sfq.ptr(keep[-1]), out_features=n, in_features=k)
    else:
        keep.append(dev(w))
        weight = sfq.new_weight(format=sfq.F32, data=sfq.ptr(keep[-1]), out_features=n, in_features=k)
    xin = x.astype(np.float64)
    if awq:
        s = oracle.to_bf16(rng.uniform(0.5, 2.0, k).astype(np.float32))
        keep.append(bf16_tensor(s))
        weight.pre_quant_scale = sfq.ptr(keep[-1])
        xin = xin * oracle.from_bf16(s).astype(np.float64)
    if convrot:
        weight.convrot, weight.convrot_group = 1, 256
        xin = (xin.reshape(rows, k // 256, 256) @ (_kron_power(4) / 16.0).T).reshape(rows, k)
    runner = sfq.LinearRunner()
    dx = dev(x)
    got = runner.forward_f32(weight, dx).cpu().numpy()
    want = xin @ w.astype(np.float64).T
    bound = 2e-6 * k * np.abs(xin).max() * np.abs(w).max() + 1e-5
    assert np.abs(got - want).max() <= bound
    ref = ref_dev()
    if ref is not None:
        ry = torch.empty((rows, n), dtype=torch.float32, device="cuda")
        rw = ref_weight_from(weight)
        ref_check(ref, ref.ref_dev_linear_forward_f32(C.byref(rw), sfq.ptr(dx), rows, sfq.ptr(ry)))
        assert np.abs(ry.cpu().numpy() - got).max() <= bound
