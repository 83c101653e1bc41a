"""The allocation-free NVFP4 Linear (sfq_linear_nvfp4_forward_static) against the runner's native path.

Collected last on purpose. Hosts that cannot allocate -- everything pre-carved by an embedder, or a call made
from inside a latency-critical callback -- use this entry point; it keeps the quantized activation in a fixed
array inside the library. The array is shared by every call and keeps old bytes, so the test makes two calls in
a row with different shapes and inputs (the second smaller, so stale bytes of the first lie right behind what
it uses) and demands bit-identical output to the regular entry point both times.
"""
import numpy as np
import pytest
import torch

import slopfab_b200 as sfq
from helpers import bf16_tensor, dev, gaussian_bf16, pack_nvfp4

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed, with_bias):
    rng = np.random.default_rng(seed)
    data, scale, g = pack_nvfp4((0.02 * rng.standard_normal((N, K))).astype(np.float32))
    bias = (0.01 * rng.standard_normal(N)).astype(np.float32) if with_bias else None
    x = bf16_tensor(gaussian_bf16((M, K), seed=seed + 1))
    return x, dev(data), dev(scale), g, (dev(bias) if with_bias else None)


def test_static_scratch_linear_matches_runner_twice_in_a_row():
    runner = sfq.LinearRunner()
    runner.set_native(True)
    for M, N, K, seed, with_bias, act in ((300, 512, 1024, 5, True, sfq.ACT_NONE), (130, 256, 320, 6, False, sfq.ACT_GELU_TANH)):
        x, d, s, g, b = _case(M, N, K, seed, with_bias)
        w = sfq.new_weight(format=sfq.NVFP4, data=sfq.ptr(d), out_features=N, in_features=K, block_scale=sfq.ptr(s),
                           global_scale=g, bias=sfq.ptr(b))
        runner.set_activation(act)
        want = runner.forward(w, x)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        sfq.check(sfq.lib.sfq_linear_nvfp4_forward_static(sfq.ptr(x), M, sfq.ptr(d), sfq.ptr(s), g, sfq.ptr(b), sfq.F32, act,
                                                          sfq.ptr(got), N, K, sfq.stream_ptr()))
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (M, N, K)
        # the kernels of the static entry point report abandoned waits in the array's own word
        assert sfq.static_status() == 0
    assert sfq.device_status() == 0


def test_static_scratch_limit_is_enforced():
    x = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    # 4096 rows x 13824 needs 28 MB + 3.5 MB of scratch: refused before anything is launched
    rc = sfq.lib.sfq_linear_nvfp4_forward_static(sfq.ptr(x), 4096, sfq.ptr(x), sfq.ptr(x), 1.0, None, sfq.F32, sfq.ACT_NONE,
                                                 sfq.ptr(x), 128, 13824, None)
    assert rc == sfq.ERR_INVALID_ARGUMENT and b"static array holds" in sfq.lib.sfq_last_error()
    assert sfq.lib.sfq_linear_nvfp4_forward_static(sfq.ptr(x), 8, sfq.ptr(x), sfq.ptr(x), 1.0, None, sfq.F32, sfq.ACT_NONE,
                                                   sfq.ptr(x), 100, 64, None) == sfq.ERR_INVALID_ARGUMENT
    # rows <= 0 is a no-op like every other forward
    assert sfq.lib.sfq_linear_nvfp4_forward_static(None, 0, None, None, 1.0, None, sfq.F32, sfq.ACT_NONE, None, 128, 64, None) == sfq.OK
