"""A small DiT block through slopfab_b200.block against a CPU composition of the oracle's pieces."""
import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import bf16_tensor, bits, dev, gaussian_bf16, pack_nvfp4
from slopfab_b200.block import BlockWeights, Nvfp4Block, Nvfp4Linear

pytestmark = pytest.mark.gpu


def _linear(n, k, rng):
    w = (0.05 * rng.standard_normal((n, k))).astype(np.float32)
    data, scale, g = pack_nvfp4(w)
    return (data, scale, g), Nvfp4Linear(dev(data), dev(scale), g, n, k)


def _cpu_attention(qkv_bits, rows, heads, hidden):
    d = hidden // heads
    qkv = oracle.from_bf16(qkv_bits).astype(np.float64)
    out = np.zeros((rows, hidden))
    for h in range(heads):
        q, k, v = (qkv[:, i * hidden + h * d: i * hidden + (h + 1) * d] for i in range(3))
        s = q @ k.T / np.sqrt(d)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h * d:(h + 1) * d] = (p / p.sum(axis=1, keepdims=True)) @ v
    return oracle.to_bf16(out.astype(np.float32))


@pytest.mark.parametrize("fuse_residual,ffn_form", [(False, "gelu"), (True, "gelu"), (False, "swiglu")])
def test_block_matches_cpu_composition(fuse_residual, ffn_form):
    rows, hidden, heads, ffn = 160, 256, 2, 512
    rng = np.random.default_rng(7)
    fc1_rows = 2 * ffn if ffn_form == "swiglu" else ffn  # the reference's H3 block: fc1 = [gate | up]
    (cq, wq), (co, wo), (c1, w1), (c2, w2) = (_linear(3 * hidden, hidden, rng), _linear(hidden, hidden, rng),
                                              _linear(fc1_rows, hidden, rng), _linear(hidden, ffn, rng))
    norm1 = oracle.to_bf16(np.ones(hidden, np.float32))
    norm2 = oracle.to_bf16((1 + 0.05 * rng.standard_normal(hidden)).astype(np.float32))
    names = ["scale_msa", "shift_msa", "gate_msa", "scale_mlp", "shift_mlp", "gate_mlp"]
    mod_h = {n: (0.1 * rng.standard_normal((3, hidden))).astype(np.float32) for n in names}
    a = (np.arange(rows) % 3).astype(np.int32)
    x = gaussian_bf16((rows, hidden), seed=8)
    weights = BlockWeights(wq, wo, w1, w2, bf16_tensor(norm1), bf16_tensor(norm2))
    mod_d = {n: dev(v) for n, v in mod_h.items()}
    block = Nvfp4Block(rows, hidden, heads, ffn, ffn_form=ffn_form)
    block.fuse_residual = fuse_residual  # gated residuals as their own kernel, or inside the GEMM epilogues
    dx = bf16_tensor(x)
    block.forward(dx, weights, mod_d, dev(a))
    torch.cuda.synchronize()
    assert sfq.device_status() == 0

    n1 = oracle.rmsnorm_bf16(x, norm1, 1e-5, mod_h["scale_msa"], mod_h["shift_msa"], a)
    qkv = oracle.nvfp4_linear(n1, cq[0], cq[1], cq[2], 3 * hidden, hidden)
    # everything up to the projections is this library's arithmetic: the stated fp4 tolerance applies
    max_abs, rel_l2, _ = oracle.compare_bf16(qkv, bits(block.qkv))
    assert max_abs <= 2e-2 and rel_l2 <= 1e-3, (max_abs, rel_l2)
    attn = _cpu_attention(qkv, rows, heads, hidden)
    branch = oracle.nvfp4_linear(attn, co[0], co[1], co[2], hidden, hidden)
    x1 = x.copy()
    oracle.lib.orc_add_gated_bf16(x1.ctypes.data, branch.ctypes.data, mod_h["gate_msa"].ctypes.data, a.ctypes.data, rows, hidden)
    n2 = oracle.rmsnorm_bf16(x1, norm2, 1e-5, mod_h["scale_mlp"], mod_h["shift_mlp"], a)
    if ffn_form == "swiglu":
        fused = oracle.nvfp4_linear(n2, c1[0], c1[1], c1[2], 2 * ffn, hidden)
        h = np.empty((rows, ffn), np.uint16)
        oracle.lib.orc_swiglu_bf16(fused.ctypes.data, rows, ffn, h.ctypes.data)
    else:
        h = oracle.nvfp4_linear(n2, c1[0], c1[1], c1[2], ffn, hidden, act=oracle.ACT_GELU_TANH)
    y2 = oracle.nvfp4_linear(h, c2[0], c2[1], c2[2], hidden, ffn)
    oracle.lib.orc_add_gated_bf16(x1.ctypes.data, y2.ctypes.data, mod_h["gate_mlp"].ctypes.data, a.ctypes.data, rows, hidden)
    # bf16 attention on the device vs fp64 on the host moves a few fp4 codes downstream: a looser, whole-block bar
    max_abs, rel_l2, corr = oracle.compare_bf16(x1, bits(dx))
    assert rel_l2 <= 3e-2 and corr > 0.999, (max_abs, rel_l2, corr)


def test_qk_norm_and_rope_run_in_place_on_the_fused_projection():
    rows, hidden, heads, ffn = 160, 256, 2, 512
    rng = np.random.default_rng(17)
    (_, wq), (_, wo), (_, w1), (_, w2) = (_linear(3 * hidden, hidden, rng), _linear(hidden, hidden, rng), _linear(ffn, hidden, rng),
                                          _linear(hidden, ffn, rng))
    ones = oracle.to_bf16(np.ones(hidden, np.float32))
    qn = oracle.to_bf16((1 + 0.1 * rng.standard_normal(128)).astype(np.float32))
    kn = oracle.to_bf16((1 + 0.1 * rng.standard_normal(128)).astype(np.float32))
    ang = rng.uniform(-3, 3, (rows, 96))
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    names = ["scale_msa", "shift_msa", "gate_msa", "scale_mlp", "shift_mlp", "gate_mlp"]
    mod = {n: dev((0.1 * rng.standard_normal((3, hidden))).astype(np.float32)) for n in names}
    a = dev((np.arange(rows) % 3).astype(np.int32))
    x = gaussian_bf16((rows, hidden), seed=18)
    plain = Nvfp4Block(rows, hidden, heads, ffn)
    plain.forward(bf16_tensor(x), BlockWeights(wq, wo, w1, w2, bf16_tensor(ones), bf16_tensor(ones)), mod, a)
    raw = bits(plain.qkv)  # the projection as the GEMM left it
    full = Nvfp4Block(rows, hidden, heads, ffn)
    y = bf16_tensor(x)
    full.forward(y, BlockWeights(wq, wo, w1, w2, bf16_tensor(ones), bf16_tensor(ones), bf16_tensor(qn), bf16_tensor(kn)), mod, a,
                 rope=(dev(cos), dev(sin)))
    torch.cuda.synchronize()
    got = bits(full.qkv)
    assert np.array_equal(got[:, :hidden], oracle.head_norm_rope(np.ascontiguousarray(raw[:, :hidden]), heads, qn, cos, sin, 1e-5))
    assert np.array_equal(got[:, hidden:2 * hidden], oracle.head_norm_rope(np.ascontiguousarray(raw[:, hidden:2 * hidden]), heads, kn, cos, sin, 1e-5))
    assert np.array_equal(got[:, 2 * hidden:], raw[:, 2 * hidden:])
    assert torch.isfinite(y.float()).all() and sfq.device_status() == 0
