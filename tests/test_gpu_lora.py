"""LoRA side branch y += (x A^T) B^T against the CPU statement of the reference's own test
(tests/test_lora_backends.cu:84-120) and against the reference's LoraRunner compiled from its sources."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import bf16_tensor, bits as bits_of
from slopfab_b200.lora import LoraRunner

pytestmark = pytest.mark.gpu

# What the reference allows its tensor-core arm against the CPU statement on this data (test_lora_backends.cu:120).
TOL = 0.00390625


def case(rows, k, rank, out_total, seed):
    x = oracle.to_bf16(oracle.make_data(rows * k, 754 + seed, 0.5)).reshape(rows, k)
    a = oracle.make_data(rank * k, 11 + seed, 0.05).reshape(rank, k)
    b = oracle.make_data(out_total * rank, 23 + seed, 0.5).reshape(out_total, rank)
    return x, a, b


def initial(rows, out):
    return oracle.to_bf16(((np.arange(rows * out) % 13) / 32).astype(np.float32)).reshape(rows, out)


@pytest.mark.parametrize("rows,k,rank,out_total,offset,out", [
    (1, 64, 8, 128, 0, 128),        # one row
    (17, 128, 4, 96, 0, 96),        # rank padded to 8 on upload
    (130, 256, 16, 384, 128, 128),  # the k third of a fused q/k/v projection
    (300, 512, 64, 256, 0, 256),    # CTA-pair kernel
    (2500, 128, 32, 128, 0, 128),   # more rows than one slice
])
def test_lora_apply_matches_the_reference_statement(rows, k, rank, out_total, offset, out):
    x, a, b = case(rows, k, rank, out_total, rows)
    y0 = initial(rows, out)
    want = oracle.from_bf16(oracle.lora_apply(x, a, b, offset, out, y0))
    runner = LoraRunner()
    runner.attach(7, a, b, offset, out)
    y = bf16_tensor(y0)
    runner.apply(7, bf16_tensor(x), y)
    runner.apply(8, bf16_tensor(x), y)  # unknown key: nothing happens
    got = oracle.from_bf16(bits_of(y))
    assert np.abs(got - want).max() <= TOL
    assert not np.array_equal(bits_of(y), y0)
    weights, scratch = runner.bytes()
    assert weights == 2 * ((rank + 7) // 8 * 8) * (k + out) and scratch > 0
    assert sfq.device_status() == 0


def test_two_factor_pairs_and_staged_upload():
    rows, k, out = 200, 256, 256
    x, a1, b1 = case(rows, k, 16, out, 1)
    _, a2, b2 = case(rows, k, 8, out, 2)
    y0 = initial(rows, out)
    want = oracle.lora_apply(x, a2, b2, 0, out, oracle.lora_apply(x, a1, b1, 0, out, y0))
    host = torch.empty(1 << 20, dtype=torch.uint8).pin_memory()
    device = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    runner = LoraRunner()
    off = runner.attach(1, a1, b1, staging=(host.data_ptr(), device.data_ptr(), 0))
    off = runner.attach(1, a2, b2, staging=(host.data_ptr(), device.data_ptr(), off))
    assert off == 16 * k * 2 + out * 16 * 2 + 8 * k * 2 + out * 8 * 2 and off % 256 == 0
    assert runner.bytes()[0] == 0  # nothing resident: the factors live in the caller's block
    device.copy_(host)
    y = bf16_tensor(y0)
    runner.apply(1, bf16_tensor(x), y)
    assert np.abs(oracle.from_bf16(bits_of(y)) - oracle.from_bf16(want)).max() <= 2 * TOL
    with pytest.raises(sfq.SfqError):
        runner.attach(2, a1, b1, 200, 100)  # slice runs past the factor
    with pytest.raises(sfq.SfqError):
        check = sfq.lib.sfq_lora_attach_staged(runner._h, C.c_void_p(3), a1.ctypes.data, b1.ctypes.data, 16, k, out, 0, out,
                                               C.c_void_p(host.data_ptr()), None, None)
        sfq.check(check)


@pytest.mark.skipif(oracle.ref is None, reason="reference build not present")
@pytest.mark.parametrize("rank", [3, 16])
@pytest.mark.parametrize("rows", [5, 64, 259])
def test_the_reference_tests_own_cases(rank, rows):
    """lora_cuda_vulkan_projection_numerics (tests/test_lora_backends.cu:169-179): in 32, out 48 in slices of 16. The
    reference's deterministic arm must equal the CPU statement bit for bit there (that pins the oracle); its tensor arm
    and ours must be within 2^-8 of it."""
    k, out_total, out = 32, 48, 16
    a = oracle.make_data(rank * k, 681, 0.125).reshape(rank, k)
    b = oracle.make_data(rank * out_total, 923, 0.125).reshape(out_total, rank)
    x = oracle.to_bf16(oracle.make_data(rows * k, 754, 0.5)).reshape(rows, k)
    y0 = initial(rows, out)
    ref = oracle.ref
    ref.ref_lora_apply.argtypes = [C.c_void_p] * 2 + [C.c_int] * 5 + [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    ref.ref_last_error.restype = C.c_char_p
    runner = LoraRunner()
    for offset in (0, 16, 32):
        want = oracle.lora_apply(x, a, b, offset, out, y0)
        got = {}
        for exact in (1, 0):
            y = bf16_tensor(y0)
            status = ref.ref_lora_apply(a.ctypes.data, b.ctypes.data, rank, k, out_total, offset, out, sfq.ptr(bf16_tensor(x)), rows,
                                        sfq.ptr(y), exact)
            assert status == 0, ref.ref_last_error().decode()
            got[exact] = bits_of(y)
        assert np.array_equal(got[1], want)
        assert np.abs(oracle.from_bf16(got[0]) - oracle.from_bf16(want)).max() <= TOL
        runner.attach(offset, a, b, offset, out)
        y = bf16_tensor(y0)
        runner.apply(offset, bf16_tensor(x), y)
        assert np.abs(oracle.from_bf16(bits_of(y)) - oracle.from_bf16(want)).max() <= TOL
    assert sfq.device_status() == 0
