"""The adaLN tables that feed the fused norm: launch_adaln_expand (bit-exact) and the fp32-compute Linear."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import RefWeight, dev, ref_check, ref_weight_from

pytestmark = pytest.mark.gpu


def _ref():
    ref = oracle.ref
    if ref is None:
        return None
    V, I = C.c_void_p, C.c_int
    ref.ref_dev_adaln_expand.argtypes = [V, V, V, V, I, I, I, I, I]
    ref.ref_dev_linear_forward_f32.argtypes = [C.POINTER(RefWeight), V, I, V]
    ref.ref_last_error.restype = C.c_char_p
    return ref


@pytest.mark.parametrize("num_t,modalities,params,channels,rank", [(1, 3, 6, 64, 16), (3, 3, 6, 320, 64), (2, 1, 2, 5120, 256)])
def test_adaln_expand_is_bit_exact(num_t, modalities, params, channels, rank):
    features = modalities * params * channels
    w = oracle.make_data(features * rank, 41, 0.2).reshape(features, rank)
    bias = oracle.make_data(features, 42, 0.5)
    code = oracle.make_data(num_t * rank, 43, 1.0).reshape(num_t, rank)
    want = oracle.adaln_expand(w, bias, code, modalities, params, channels)
    dw, db, dc = dev(w), dev(bias), dev(code)
    out = torch.empty(want.shape, dtype=torch.float32, device="cuda")
    sfq.check(sfq.lib.sfq_adaln_expand(sfq.ptr(dw), sfq.ptr(db), sfq.ptr(dc), sfq.ptr(out), num_t, modalities, params, channels, rank,
                                       sfq.stream_ptr()))
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # row p = (modality * params + param) * channels + channel of the Linear lands at [param, t, modality, channel]
    p = (1 % modalities * params + 1) * channels + 5
    acc = np.float32(bias[p])
    for k in range(rank):
        acc = np.float32(np.float64(w[p, k]) * np.float64(code[0, k]) + np.float64(acc))  # fma: one rounding
    assert got[1, 0, 1 % modalities, 5] == acc
    ref = _ref()
    if ref is not None:
        rout = torch.empty_like(out)
        ref_check(ref, ref.ref_dev_adaln_expand(sfq.ptr(dw), sfq.ptr(db), sfq.ptr(dc), sfq.ptr(rout), num_t, modalities, params,
                                                channels, rank))
        assert torch.equal(rout, out)


def test_adaln_expand_refusals():
    t = torch.zeros(16, dtype=torch.float32, device="cuda")
    for args in [(0, 1, 1, 4, 4), (1, 1, 1, 4, 0), (70000, 1, 1, 4, 4)]:
        with pytest.raises(sfq.SfqError, match="launch_adaln_expand"):
            sfq.check(sfq.lib.sfq_adaln_expand(sfq.ptr(t), sfq.ptr(t), sfq.ptr(t), sfq.ptr(t), *args, None))


@pytest.mark.parametrize("fmt", ["f32", "bf16"])
@pytest.mark.parametrize("rows,n,k", [(1, 192, 64), (3, 1000, 256), (70, 130, 100)])
def test_forward_f32_against_the_fp64_product(fmt, rows, n, k):
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = (0.05 * rng.standard_normal((n, k))).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    if fmt == "bf16":
        wbits = oracle.to_bf16(w)
        w = oracle.from_bf16(wbits)
        dw = dev(wbits)
        weight = sfq.new_weight(format=sfq.BF16, data=sfq.ptr(dw), out_features=n, in_features=k)
    else:
        dw = dev(w)
        weight = sfq.new_weight(format=sfq.F32, data=sfq.ptr(dw), out_features=n, in_features=k)
    db = dev(bias)
    weight.bias = sfq.ptr(db)
    weight.bias_format = sfq.F32
    runner = sfq.LinearRunner()
    dx = dev(x)
    got = runner.forward_f32(weight, dx).cpu().numpy()
    want = x.astype(np.float64) @ w.astype(np.float64).T + bias
    # fp32 accumulation over k terms of magnitude ~|x||w|: a few ulps of the largest partial sum
    assert np.abs(got - want).max() <= 2e-6 * k * np.abs(x).max() * np.abs(w).max() + 1e-6
    ref = _ref()
    if ref is not None:
        ry = torch.empty((rows, n), dtype=torch.float32, device="cuda")
        rw = ref_weight_from(weight)
        ref_check(ref, ref.ref_dev_linear_forward_f32(C.byref(rw), sfq.ptr(dx), rows, sfq.ptr(ry)))
        assert np.abs(ry.cpu().numpy() - got).max() <= 2e-6 * k * np.abs(x).max() * np.abs(w).max() + 1e-6


def test_forward_f32_refuses_what_it_does_not_build():
    t = torch.zeros(256 * 256, dtype=torch.float32, device="cuda")
    runner = sfq.LinearRunner()
    w = sfq.new_weight(format=sfq.W4A8, data=sfq.ptr(t), out_features=256, in_features=256)
    with pytest.raises(sfq.SfqError, match="BF16 activations"):
        runner.forward_f32(w, t.view(256, 256))
