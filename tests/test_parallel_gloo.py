"""world_size-2 gloo runs of the multi-GPU host logic on CPU: row/column sharding and the single all-gather of
the column-split variant, with the CPU oracle standing in for the device kernels (tests only)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from slopfab_b200.parallel import all_gather_rows, column_shard, column_split_int8_forward, row_chunks, token_shard


def test_shard_arithmetic():
    for rows in (0, 1, 7, 111600, 4096):
        for world in (1, 2, 4, 8):
            blocks = [token_shard(rows, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and sum(c for _, c in blocks) == rows
            assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1
    assert token_shard(111600, 8, 3) == (3 * 13950, 13950)
    cols = [column_shard(13824, 8, r) for r in range(8)]
    assert sum(c for _, c in cols) == 13824 and all(s % 128 == 0 and c % 128 == 0 for s, c in cols)


def test_row_chunks_are_aligned_and_cover_the_rows():
    for rows in (1, 127, 128, 129, 1000, 13950, 55800):
        for chunks in (1, 2, 3, 4):
            pieces = row_chunks(rows, chunks)
            assert pieces[0][0] == 0 and sum(c for _, c in pieces) == rows and len(pieces) <= chunks
            assert all(pieces[i][0] + pieces[i][1] == pieces[i + 1][0] for i in range(len(pieces) - 1))
            assert all(r0 % 128 == 0 for r0, _ in pieces)
    assert row_chunks(13950, 2) == [(0, 7040), (7040, 6910)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 37, 256, 512  # ragged: 19 + 18 rows
        rng = np.random.default_rng(0)
        x = oracle.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        w8 = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
        cs = (rng.random(N) * 0.01 + 1e-3).astype(np.float32)
        r0, rc = token_shard(M, world, rank)
        c0, cc = column_shard(N, world, rank)

        def quantize(x_local):
            q, s = oracle.quantize_int8_token(oracle.convrot_bf16(np.ascontiguousarray(x_local.numpy().view(np.uint16))))
            return torch.from_numpy(q), torch.from_numpy(s)

        def gemm(q_all, s_all):
            acc = oracle.int8_gemm(q_all.numpy(), np.ascontiguousarray(w8[c0:c0 + cc]))
            y = np.empty((q_all.shape[0], cc), np.uint16)
            oracle.lib.orc_w4a8_output_bf16(acc.ctypes.data, s_all.numpy().ctypes.data, np.ascontiguousarray(cs[c0:c0 + cc]).ctypes.data,
                                            q_all.shape[0], cc, y.ctypes.data)
            return torch.from_numpy(y.view(np.int16))

        x_local = torch.from_numpy(x[r0:r0 + rc].view(np.int16))
        y_cols = column_split_int8_forward(quantize, gemm, x_local)
        # gather the column blocks for the check (not part of the path)
        full = all_gather_rows(y_cols.t().contiguous()).t().contiguous()
        q_ref, s_ref = oracle.quantize_int8_token(oracle.convrot_bf16(x))
        want = np.empty((M, N), np.uint16)
        acc = oracle.int8_gemm(q_ref, w8)
        oracle.lib.orc_w4a8_output_bf16(acc.ctypes.data, s_ref.ctypes.data, cs.ctypes.data, M, N, want.ctypes.data)
        ok = np.array_equal(full.numpy().view(np.uint16), want)
        # token sharding: concatenating the ranks' rows reproduces the unsharded result, no collective needed
        rows = all_gather_rows(torch.from_numpy(want[r0:r0 + rc].view(np.int16)))
        ok = ok and np.array_equal(rows.numpy().view(np.uint16), want)
        if rank == 0:
            out.put(bool(ok))
    finally:
        dist.destroy_process_group()


def test_column_split_and_token_sharding_world2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout=120)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join()
    assert [p.exitcode for p in procs] == [0, 0]
    assert out.get(timeout=5) is True
