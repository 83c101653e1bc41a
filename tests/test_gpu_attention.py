"""Full self-attention (head_dim 128) against the dense fp64 softmax of the reference's test fixture, on the
reference's own shapes, seeds and bound (tests/test_nn_kernels_attention_synthetic.cu:4-160)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import slopfab_b200 as sfq
from helpers import bf16_tensor, bits

pytestmark = pytest.mark.gpu
D = 128


def attention(q, k, v, heads, kv_heads, out=None, scale=0.0, ld_q=None, ld_kv=None):
    """q: bf16 [seq_q, >= heads*128] tensors (views allowed); returns out [seq_q, heads*128]."""
    seq_q, seq_kv = q.shape[0], k.shape[0]
    out = torch.empty((seq_q, heads * D), dtype=torch.bfloat16, device="cuda") if out is None else out
    n = C.c_size_t()
    sfq.check(sfq.lib.sfq_attention_workspace_bytes(seq_kv, kv_heads, D, C.byref(n)))
    ws = torch.empty(n.value, dtype=torch.uint8, device="cuda")
    sfq.check(sfq.lib.sfq_attention_forward(q.data_ptr(), ld_q or q.stride(0), k.data_ptr(), v.data_ptr(), ld_kv or k.stride(0),
                                            out.data_ptr(), out.stride(0), seq_q, seq_kv, heads, kv_heads, D, scale, ws.data_ptr(), n.value,
                                            sfq.stream_ptr()))
    return out


def data(seq, heads, seed, scale):
    return oracle.from_bf16(oracle.to_bf16(oracle.make_data(seq * heads * D, seed, scale))).reshape(seq, heads * D)


def close(want, got):
    err = np.abs(got - want)
    bound = 1e-3 + 1e-2 * np.abs(want)
    assert (err <= bound).all(), (float(err.max()), int(np.argmax(err - bound)))


def run_case(q, k, v, heads, kv_heads):
    want = oracle.attention(q, k, v, heads, kv_heads, D, 1.0 / np.sqrt(D))
    out = attention(bf16_tensor(oracle.to_bf16(q)), bf16_tensor(oracle.to_bf16(k)), bf16_tensor(oracle.to_bf16(v)), heads, kv_heads)
    close(want, oracle.from_bf16(bits(out)))
    assert sfq.device_status() == 0
    return out


def test_reference_blocked_case():
    run_case(data(512, 4, 161, 0.3), data(512, 4, 162, 0.3), data(512, 4, 163, 1.0), 4, 4)


@pytest.mark.parametrize("seq", [17, 61, 127, 199])
def test_ragged_tail(seq):
    run_case(data(seq, 3, 401 + seq, 0.3), data(seq, 3, 402 + seq, 0.3), data(seq, 3, 403 + seq, 1.0), 3, 3)


@pytest.mark.parametrize("seq", [1, 127, 128, 259, 2051])
def test_compact_query_chunks_equal_the_full_call(seq):
    q, k, v = data(seq, 2, 9701, 0.3), data(seq, 2, 9702, 0.3), data(seq, 2, 9703, 1.0)
    full = run_case(q, k, v, 2, 2)
    dq, dk, dv = (bf16_tensor(oracle.to_bf16(t)) for t in (q, k, v))
    for chunk in (64, 257):
        parts = [attention(dq[s:s + chunk], dk, dv, 2, 2) for s in range(0, seq, chunk)]
        assert torch.equal(torch.cat(parts), full)  # a query row never depends on which chunk carried it


def test_grouped_heads_and_fused_projection_views():
    seq, heads, kv_heads = 300, 8, 2
    q, k, v = data(seq, heads, 51, 0.3), data(seq, kv_heads, 52, 0.3), data(seq, kv_heads, 53, 1.0)
    run_case(q, k, v, heads, kv_heads)
    # q, k, v as the thirds of one [seq, 3 * heads * 128] buffer, as the fused QKV projection leaves them
    heads = 3
    q, k, v = data(seq, heads, 61, 0.3), data(seq, heads, 62, 0.3), data(seq, heads, 63, 1.0)
    fused = bf16_tensor(oracle.to_bf16(np.concatenate([q, k, v], axis=1)))
    w = heads * D
    out = attention(fused[:, :w], fused[:, w:2 * w], fused[:, 2 * w:], heads, heads)
    close(oracle.attention(q, k, v, heads, heads, D, 1.0 / np.sqrt(D)), oracle.from_bf16(bits(out)))


def test_running_maximum_that_keeps_growing():
    """Keys grow along the sequence so that every few tiles the maximum jumps by more than the rescale threshold: the
    accumulator rescale in tensor memory runs many times."""
    seq, heads = 1500, 2
    q = data(seq, heads, 71, 1.0)
    ramp = (0.2 + 3.0 * np.arange(seq) / seq).astype(np.float32)[:, None]
    sign = np.sign(q[0:1])
    sign[sign == 0] = 1
    k = oracle.from_bf16(oracle.to_bf16(sign * ramp))  # q[0] . k[j] = ramp[j] * sum |q[0]|: grows along the sequence
    v = data(seq, heads, 73, 1.0)
    want = oracle.attention(q, k, v, heads, heads, D, 1.0 / np.sqrt(D))
    out = attention(bf16_tensor(oracle.to_bf16(q)), bf16_tensor(oracle.to_bf16(k)), bf16_tensor(oracle.to_bf16(v)), heads, heads)
    close(want, oracle.from_bf16(bits(out)))
    scores = (q[0, :D] @ k[:, :D].T) / np.sqrt(D) * np.log2(np.e)
    assert scores.max() - scores[:128].max() > 16  # row 0 crosses the threshold at least twice
    assert sfq.device_status() == 0


def test_against_torch_on_a_longer_sequence():
    torch.manual_seed(5)
    seq, heads = 4096 + 77, 4
    q, k, v = (torch.randn(seq, heads * D, device="cuda").mul_(s).to(torch.bfloat16) for s in (1.0, 1.0, 1.0))
    out = attention(q, k, v, heads, heads)
    sh = lambda t: t.view(seq, heads, D).transpose(0, 1).float()  # noqa: E731
    want = torch.nn.functional.scaled_dot_product_attention(sh(q), sh(k), sh(v)).transpose(0, 1).reshape(seq, heads * D)
    err = (out.float() - want).abs()
    assert bool((err <= 1e-3 + 1e-2 * want.abs()).all()), float(err.max())
    assert sfq.device_status() == 0


def test_refusals():
    t = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(sfq.SfqError, match="head_dim"):
        sfq.check(sfq.lib.sfq_attention_forward(t.data_ptr(), 64, t.data_ptr(), t.data_ptr(), 64, t.data_ptr(), 64, 128, 128, 1, 1, 64, 0.0,
                                                t.data_ptr(), 1 << 20, None))
    o = torch.zeros_like(t)
    with pytest.raises(sfq.SfqError, match="workspace"):
        sfq.check(sfq.lib.sfq_attention_forward(t.data_ptr(), 128, t.data_ptr(), t.data_ptr(), 128, o.data_ptr(), 128, 128, 128, 1, 1, 128, 0.0,
                                                t.data_ptr(), 16, None))
    with pytest.raises(sfq.SfqError, match="alias"):
        sfq.check(sfq.lib.sfq_attention_forward(t.data_ptr(), 128, t.data_ptr(), t.data_ptr(), 128, t.data_ptr(), 128, 128, 128, 1, 1, 128, 0.0,
                                                o.data_ptr(), 1 << 16, None))
