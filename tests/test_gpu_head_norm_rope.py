"""QK-norm over the head dimension followed by MM-RoPE, in place on the thirds of a fused projection: bit-exact
against the CPU restatement and against the reference's two kernels (launch_head_rmsnorm, launch_rope_h3)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import bf16_tensor, bits, dev, ref_check

pytestmark = pytest.mark.gpu


def tables(rows, seed):
    ang = oracle.make_data(rows * 96, seed, 3.0).reshape(rows, 96)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    cos[0, :4] = [0.0, 1e-40, -1e-39, 1.0]  # zeros and subnormals: the canonicalisation paths
    sin[0, :4] = [1.0, 1e-39, 0.0, -0.0]
    return cos, sin


def run(x_bits, ld, heads, w=None, cos=None, sin=None, eps=1e-6):
    t = bf16_tensor(x_bits)
    keep = [dev(a) if a is not None else None for a in (w, cos, sin)]
    p = [sfq.ptr(a) if a is not None else None for a in keep]
    sfq.check(sfq.lib.sfq_head_norm_rope(sfq.ptr(t), ld, p[0], p[1], p[2], x_bits.shape[0], heads, 128, eps, sfq.stream_ptr()))
    return bits(t)


@pytest.mark.parametrize("rows,heads", [(1, 1), (37, 3), (300, 40)])
@pytest.mark.parametrize("what", ["norm", "rope", "both"])
def test_bit_exact_against_oracle_and_reference(rows, heads, what):
    x = oracle.to_bf16(oracle.make_data(rows * heads * 128, 71 + rows, 2.0)).reshape(rows, heads * 128)
    x[0, :8] = [0x0001, 0x8001, 0x0000, 0x8000, 0x007F, 0x3F80, 0x0080, 0xBF80]  # bf16 subnormals, zeros, ones
    w = oracle.to_bf16(1.0 + oracle.make_data(128, 5, 0.2)) if what != "rope" else None
    cos, sin = tables(rows, 9) if what != "norm" else (None, None)
    want = oracle.head_norm_rope(x, heads, w, cos, sin, 1e-6)
    got = run(x, heads * 128, heads, w, cos, sin)
    assert np.array_equal(got, want)
    if what != "norm":
        assert np.array_equal(got[:, 96:128], (oracle.head_norm_rope(x, heads, w, None, None, 1e-6) if w is not None else x)[:, 96:128])
    ref = oracle.ref
    if ref is not None:
        ref.ref_dev_head_norm_rope.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_float]
        ref.ref_last_error.restype = C.c_char_p
        t = bf16_tensor(x)
        keep = [dev(a) if a is not None else None for a in (w, cos, sin)]
        p = [sfq.ptr(a) if a is not None else None for a in keep]
        ref_check(ref, ref.ref_dev_head_norm_rope(sfq.ptr(t), p[0], p[1], p[2], rows, heads, 128, 1e-6))
        assert np.array_equal(bits(t), want)  # pins the restatement
    assert sfq.device_status() == 0


def test_thirds_of_a_fused_projection_in_place():
    rows, heads = 130, 4
    w = heads * 128
    fused = oracle.to_bf16(oracle.make_data(rows * 3 * w, 3, 1.5)).reshape(rows, 3 * w)
    qn, kn = oracle.to_bf16(1.0 + oracle.make_data(128, 6, 0.1)), oracle.to_bf16(1.0 + oracle.make_data(128, 7, 0.1))
    cos, sin = tables(rows, 11)
    t = bf16_tensor(fused)
    dq, dk, dc, ds = dev(qn), dev(kn), dev(cos), dev(sin)
    base = t.data_ptr()
    for third, wt in ((0, dq), (1, dk)):
        sfq.check(sfq.lib.sfq_head_norm_rope(base + third * w * 2, 3 * w, sfq.ptr(wt), sfq.ptr(dc), sfq.ptr(ds), rows, heads, 128, 1e-6,
                                             sfq.stream_ptr()))
    got = bits(t)
    assert np.array_equal(got[:, :w], oracle.head_norm_rope(np.ascontiguousarray(fused[:, :w]), heads, qn, cos, sin, 1e-6))
    assert np.array_equal(got[:, w:2 * w], oracle.head_norm_rope(np.ascontiguousarray(fused[:, w:2 * w]), heads, kn, cos, sin, 1e-6))
    assert np.array_equal(got[:, 2 * w:], fused[:, 2 * w:])  # v is never touched


def test_refusals():
    t = torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(sfq.SfqError, match="head_dim 128"):
        sfq.check(sfq.lib.sfq_head_norm_rope(sfq.ptr(t), 64, sfq.ptr(t), None, None, 4, 1, 64, 1e-6, None))
    with pytest.raises(sfq.SfqError, match="nothing to do"):
        sfq.check(sfq.lib.sfq_head_norm_rope(sfq.ptr(t), 128, None, None, None, 4, 1, 128, 1e-6, None))
    with pytest.raises(sfq.SfqError, match="row pitch"):
        sfq.check(sfq.lib.sfq_head_norm_rope(sfq.ptr(t), 64, sfq.ptr(t), None, None, 4, 1, 128, 1e-6, None))
