"""Two-GPU runs of the multi-GPU variants (skipped on a single GPU): token sharding and the FFN-up column
split with its single NCCL all-gather must reproduce the one-GPU result bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import oracle
    import slopfab_b200 as sfq
    from helpers import bf16_tensor, dev, gaussian_bf16, synthetic_packed_int8
    from slopfab_b200.parallel import ColumnSplitPlan, column_shard, column_split_w4a8_forward, token_shard
    from helpers import pack_nvfp4

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        M, N, K = 1000, 1536, 1024  # ragged token split, column blocks of 768
        packed, s_rel, s_ch, book = synthetic_packed_int8(4, 16, N, K, seed=5)
        bias = (0.01 * np.random.default_rng(6).standard_normal(N)).astype(np.float32)
        x = gaussian_bf16((M, K), seed=7, outliers=True)
        keep = [dev(packed), dev(s_rel), dev(s_ch), dev(book), dev(bias)]
        w = sfq.new_weight(format=sfq.W4A8, data=sfq.ptr(keep[0]), out_features=N, in_features=K, block_scale=sfq.ptr(keep[1]),
                           weight_scale=sfq.ptr(keep[2]), w4_codebook=sfq.ptr(keep[3]), packed_group_size=16, convrot=1,
                           convrot_group=256, bias=sfq.ptr(keep[4]))
        full = sfq.LinearRunner().forward(w, bf16_tensor(x))          # what one GPU computes
        r0, rc = token_shard(M, world, rank)
        c0, cc = column_shard(N, world, rank)
        w8 = torch.empty((N, K), dtype=torch.int8, device="cuda")
        sfq.check(sfq.lib.sfq_unpack_w4a8_int8(sfq.ptr(keep[0]), sfq.ptr(keep[1]), sfq.ptr(keep[3]), sfq.ptr(w8), N, K, 16,
                                               sfq.stream_ptr()))
        y_cols = column_split_w4a8_forward(bf16_tensor(np.ascontiguousarray(x[r0:r0 + rc])), w8[c0:c0 + cc].contiguous(),
                                           keep[2][c0:c0 + cc].contiguous(), keep[4][c0:c0 + cc].contiguous())
        torch.cuda.synchronize()
        ok = torch.equal(y_cols.view(torch.int16), full[:, c0:c0 + cc].contiguous().view(torch.int16))
        # token sharding: this rank's rows through the ordinary runner equal the same rows of the full result
        mine = sfq.LinearRunner().forward(w, bf16_tensor(np.ascontiguousarray(x[r0:r0 + rc])))
        ok = ok and torch.equal(mine.view(torch.int16), full[r0:r0 + rc].view(torch.int16))
        # the preallocated plan (equal token counts per rank): int8 and fp4 activations, one all-gather each
        import ctypes as C
        Me = 1024
        xe = gaussian_bf16((Me, K), seed=9)
        me = Me // world
        xl = bf16_tensor(np.ascontiguousarray(xe[rank * me:(rank + 1) * me]))
        plans = {p: ColumnSplitPlan("w4a8", me, K, cc, (w8[c0:c0 + cc].contiguous(), keep[2][c0:c0 + cc].contiguous()), world, pipeline=p)
                 for p in ("overlap", "blocking")}
        got = plans["overlap"].forward(xl)
        q = torch.empty((Me, K), dtype=torch.int8, device="cuda")
        rs = torch.empty(Me, device="cuda")
        xa = bf16_tensor(xe)
        sfq.check(sfq.lib.sfq_quantize_int8_token(sfq.ptr(xa), None, sfq.ptr(q), sfq.ptr(rs), None, Me, K, 1, sfq.stream_ptr()))
        want = torch.empty((Me, N), dtype=torch.bfloat16, device="cuda")
        ep = sfq.Epilogue(sfq.ptr(rs), sfq.ptr(keep[2]), 1.0, None, sfq.F32, sfq.ACT_NONE)
        sfq.check(sfq.lib.sfq_gemm_int8(sfq.ptr(q), sfq.ptr(w8), C.byref(ep), sfq.ptr(want), Me, N, K, sfq.stream_ptr()))
        torch.cuda.synchronize()
        ok = ok and torch.equal(got.view(torch.int16), want[:, c0:c0 + cc].contiguous().view(torch.int16))
        # both pipelines, and each a second time over its own buffers (the gather slots and events are reused)
        for p in ("overlap", "blocking", "overlap"):
            again = plans[p].forward(xl)
            torch.cuda.synchronize()
            ok = ok and torch.equal(again.view(torch.int16), want[:, c0:c0 + cc].contiguous().view(torch.int16))
        wf = (0.02 * np.random.default_rng(10).standard_normal((N, K))).astype(np.float32)
        data, scale, gs = pack_nvfp4(wf)
        dd, ds = dev(data), dev(scale)
        plan4 = ColumnSplitPlan("nvfp4", me, K, cc, (dd[c0:c0 + cc].contiguous(),
                                                     ds.view(N // 128, -1)[c0 // 128:(c0 + cc) // 128].contiguous().view(-1), gs), world)
        got4 = plan4.forward(xl)
        got4 = plan4.forward(xl)  # second call: slots rewritten while the previous call's events are still around
        xq = torch.empty((Me, K // 2), dtype=torch.uint8, device="cuda")
        xs = torch.empty(sfq.lib.sfq_nvfp4_act_scale_bytes(Me, K), dtype=torch.uint8, device="cuda")
        sfq.check(sfq.lib.sfq_quantize_nvfp4_block(sfq.ptr(xa), None, sfq.ptr(xq), sfq.ptr(xs), None, Me, K,
                                                   sfq.NVFP4_ACT_GEMM_FEED, sfq.stream_ptr()))
        want4 = torch.empty((Me, N), dtype=torch.bfloat16, device="cuda")
        ep4 = sfq.Epilogue(None, None, gs, None, sfq.F32, sfq.ACT_NONE)
        sfq.check(sfq.lib.sfq_gemm_nvfp4(sfq.ptr(xq), sfq.ptr(xs), sfq.ptr(dd), sfq.ptr(ds), C.byref(ep4), sfq.ptr(want4), Me, N, K,
                                         sfq.stream_ptr()))
        torch.cuda.synchronize()
        ok = ok and torch.equal(got4.view(torch.int16), want4[:, c0:c0 + cc].contiguous().view(torch.int16))
        ok = ok and sfq.device_status() == 0
        flag = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            out.put(bool(flag.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_split_and_token_sharding_on_two_gpus():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout=300)
    finally:
        # a worker that is still alive holds its GPU and its communicator: end it before the verdict
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join()
    assert [p.exitcode for p in procs] == [0, 0]
    assert out.get(timeout=5) is True
