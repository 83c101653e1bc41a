"""The abort path of the CTA-pair GEMMs: a bounded wait that runs out must end the launch by itself.

Every barrier wait in the GEMM kernels has a limit; past it a thread records a status code, raises its CTA's abort
flag, the producer lets the copies in flight land, the accumulator memory (TMEM) is handed back and the kernel
returns. Nothing in normal operation ever takes that path, so this test makes one wait run out on purpose, the
harmless way: a test hook tells the producer warp to announce the bytes of one pipeline stage and then not issue
its loads, and shortens the limit from about a second to a few tens of milliseconds. The barrier of that stage can
then never complete. No trap, no bad address, no endless loop: the kernels leave through their own exit.

Checked: the launch returns, the status word holds one of the kernel's wait codes and reads as zero afterwards, and a
second, ordinary launch of the same shape (which needs all 512 TMEM columns of every SM again) is bit-exact.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import P, bits, dev
from test_gpu_gemm import _nvfp4_case

pytestmark = pytest.mark.gpu

WAIT_CYCLES = 1 << 25  # ~20 ms at the clocks these kernels run at; the longest legitimate wait here is microseconds


def _int8_launch(M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    rs = np.full(M, 2.0 ** -6, np.float32)
    cs = np.full(N, 2.0 ** -7, np.float32)
    keep = [dev(a), dev(w), dev(rs), dev(cs)]
    y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ep = sfq.Epilogue(sfq.ptr(keep[2]), sfq.ptr(keep[3]), 1.0, None, sfq.F32, sfq.ACT_NONE)
    want = np.empty((M, N), np.uint16)
    acc = oracle.int8_gemm(a, w)
    oracle.lib.orc_w4a8_output_bf16(P(acc), P(rs), P(cs), M, N, P(want))

    def launch():
        sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(keep[0]), sfq.ptr(keep[1]), C.byref(ep), sfq.ptr(y), M, N, K, None))
        return y

    return launch, want, keep


def _nvfp4_launch(M, N, K, seed):
    x, data, scale, g = _nvfp4_case(M, N, K, seed=seed)
    from helpers import bf16_tensor
    dx = bf16_tensor(x)
    xq = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda")
    xs = torch.empty(sfq.lib.sfq_nvfp4_act_scale_bytes(M, K), dtype=torch.uint8, device="cuda")
    sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(dx), None, sfq.ptr(xq), sfq.ptr(xs), None, M, K, sfq.NVFP4_ACT_GEMM_FEED, None))
    keep = [dev(data), dev(scale), xq, xs]
    y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ep = sfq.Epilogue(None, None, g, None, sfq.F32, sfq.ACT_NONE)
    want = oracle.nvfp4_linear(x, data, scale, g, N, K)

    def launch():
        sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(xq), sfq.ptr(xs), sfq.ptr(keep[0]), sfq.ptr(keep[1]), C.byref(ep), sfq.ptr(y), M, N, K, None))
        return y

    return launch, want, keep


@pytest.mark.parametrize("kind", ["int8", "nvfp4"])
def test_a_lost_load_ends_through_the_abort_path(kind):
    M, N, K = 512, 512, 2048  # CTA-pair kernel, four tiles, 16 (int8) or 8 (fp4) pipeline stages per tile
    launch, want, keep = (_int8_launch if kind == "int8" else _nvfp4_launch)(M, N, K, seed=11)
    assert sfq.device_status() == 0
    sfq.lib.sfq_test_gemm_lost_load(5, WAIT_CYCLES)  # every pair's sixth stage never arrives
    try:
        launch()
        torch.cuda.synchronize()  # returns: the kernel ended by itself
    finally:
        sfq.lib.sfq_test_gemm_lost_load(-1, 0)
    code = sfq.device_status()
    assert 1 <= code <= 6, f"expected one of the kernels' wait codes, got {code}"
    assert sfq.device_status() == 0  # reading cleared it
    # an ordinary launch right afterwards: the accumulator memory was handed back, nothing is left armed
    y = launch()
    torch.cuda.synchronize()
    assert sfq.device_status() == 0
    if kind == "int8":
        assert np.array_equal(bits(y), want)
    else:
        max_abs, rel_l2, _ = oracle.compare_bf16(want, bits(y))
        assert max_abs <= 2e-2 and rel_l2 <= 1e-3
