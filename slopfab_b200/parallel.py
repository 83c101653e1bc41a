"""Multi-GPU execution of the quantized Linear: one process per GPU, torch.distributed for the plumbing.

Every output row of the path depends on one input row, and weights are read-only, so:

* token sharding (primary): rank r owns a contiguous block of token rows and a full replica of the packed
  weights; there is no collective on the data path.
* FFN-up column split (secondary): rank r owns output columns [c0, c1) of the weight. The *quantized*
  activation -- the smallest representation of x (int8 + one fp32 scale per row) -- is exchanged with ONE
  all-gather, landing in ordinary local memory, and each rank then computes y[:, c0:c1] for all tokens.

The reference is single-GPU (no collective exists in its tree); this file is new behaviour.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def token_shard(rows: int, world: int, rank: int) -> tuple[int, int]:
    """(first row, row count) of rank's contiguous block; the first rows % world ranks take one extra row."""
    if rows < 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("token_shard: bad arguments")
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def column_shard(cols: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """(first column, column count) in units of `multiple` columns (128 keeps NVFP4 scale tiles whole)."""
    if cols % multiple != 0:
        raise ValueError(f"column_shard: {cols} columns are not a multiple of {multiple}")
    start, count = token_shard(cols // multiple, world, rank)
    return start * multiple, count * multiple


def all_gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenates every rank's rows (ragged counts allowed) with a single all-gather of padded blocks."""
    if local.dtype != torch.uint8:  # move bytes: every backend gathers uint8, not every backend gathers int16/bf16
        width = local.shape[1:]
        flat = local.contiguous().view(local.shape[0], -1).view(torch.uint8)
        return all_gather_rows(flat, group).view(local.dtype).view((-1,) + tuple(width))
    world = dist.get_world_size(group)
    counts = torch.zeros(world, dtype=torch.int64, device=local.device)
    counts[dist.get_rank(group)] = local.shape[0]
    dist.all_reduce(counts, group=group)
    counts = counts.tolist()
    most = max(counts)
    padded = local
    if local.shape[0] != most:
        padded = torch.zeros((most,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded[: local.shape[0]] = local
    out = torch.empty((world * most,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    if all(c == most for c in counts):
        return out
    return torch.cat([out[r * most: r * most + counts[r]] for r in range(world)], dim=0)


def column_split_int8_forward(quantize, gemm, x_local: torch.Tensor, group=None) -> torch.Tensor:
    """y[:, local columns] for ALL tokens.

    quantize(x_local) -> (q int8 [m, K], row_scale fp32 [m]) runs on the local token rows;
    gemm(q_all, row_scale_all) -> y_all_tokens[:, local columns] runs against the local weight columns.
    The one collective is the all-gather of q with the row scales appended as four extra int8 columns.
    """
    q, s = quantize(x_local)
    packed = torch.cat([q, s.view(-1, 1).contiguous().view(torch.int8).view(-1, 4)], dim=1)
    gathered = all_gather_rows(packed, group)
    k = q.shape[1]
    q_all = gathered[:, :k].contiguous()
    s_all = gathered[:, k:].contiguous().view(torch.float32).view(-1)
    return gemm(q_all, s_all)


def column_split_w4a8_forward(x_local: torch.Tensor, w8_cols: torch.Tensor, col_scale: torch.Tensor,
                              bias: torch.Tensor | None = None, activation: int = 0, group=None) -> torch.Tensor:
    """FFN-up column split on GPUs, W4A8/W6A8 flavour.

    x_local  bf16 [m_local, K]   this rank's token rows
    w8_cols  int8 [n_local, K]   this rank's output columns of the expanded weight (sfq_unpack_w4a8_int8 / w6a8)
    col_scale fp32 [n_local], bias fp32 [n_local] or None
    Returns bf16 [M_total, n_local]: this rank's columns for ALL tokens. One NCCL all-gather (of the int8
    activation with its row scales appended) is the only collective; the GEMM reads local memory only.
    """
    import ctypes as C

    from . import F32, Epilogue, check, lib, ptr, stream_ptr

    m, k = x_local.shape
    n = w8_cols.shape[0]

    def quantize(x):
        q = torch.empty((m, k), dtype=torch.int8, device=x.device)
        s = torch.empty(m, dtype=torch.float32, device=x.device)
        check(lib.sfq_quantize_int8_token(ptr(x), None, ptr(q), ptr(s), None, m, k, 1, stream_ptr()))
        return q, s

    def gemm(q_all, s_all):
        rows = q_all.shape[0]
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=q_all.device)
        ep = Epilogue(ptr(s_all), ptr(col_scale), 1.0, ptr(bias), F32, activation)
        check(lib.sfq_gemm_int8(ptr(q_all), ptr(w8_cols), C.byref(ep), ptr(y), rows, n, k, stream_ptr()))
        return y

    return column_split_int8_forward(quantize, gemm, x_local.contiguous(), group)


def exchange_steps(world: int, rank: int) -> list[tuple[int, int]]:
    """The all-gather of one block per rank as world - 1 pairwise steps: in step s (1-based) this rank sends its own
    block to rank + s and receives the block of rank - s (mod world). Every rank sends and receives exactly one block
    per step, so all links are busy in every step, and after step s a rank holds the blocks of s + 1 sources."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("exchange_steps: bad arguments")
    return [((rank + s) % world, (rank - s) % world) for s in range(1, world)]


def gather_blocks_stepwise(blocks: list[torch.Tensor], rank: int, group=None, on_block=None) -> None:
    """Fills blocks[src] for every src != rank from the rank that owns it (blocks[rank] is this rank's own, already
    written), one exchange_steps step at a time. on_block(src) is called after the step that delivered blocks[src] has
    been waited for: on CUDA tensors that wait only orders the CURRENT stream behind the transfer (the host runs
    on), so the caller can record an event there and release that block's consumer while later steps are still moving."""
    world = len(blocks)
    for dst, src in exchange_steps(world, rank):
        ops = [dist.P2POp(dist.isend, blocks[rank], dst, group), dist.P2POp(dist.irecv, blocks[src], src, group)]
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        if on_block is not None:
            on_block(src)


class ColumnSplitPlan:
    """FFN-up column split with preallocated buffers and equal token counts per rank (the benchmark's case).

    Every rank quantizes its own `m` token rows into one block [quantized rows | their scales]; the blocks of all ranks
    are brought into ordinary local memory (the one all-gather of the scheme) and the local weight columns are
    multiplied block by block, one GEMM launch per source rank, so no block waits for a repack. Kinds: "w4a8" (int8 rows
    + fp32 row scales; `weight` = (int8 [n_local, K], col_scale fp32 [n_local])) and "nvfp4" (fp4 rows + 128x4-tiled
    e4m3 scales; `weight` = (u8 [n_local, K/2], tiled scales, global_scale)).

    pipeline="overlap" (default): the rank's own block is multiplied at once, while a communication stream runs the
      gather as exchange_steps' pairwise steps; one event per delivered block releases that block's GEMM, so the
      transfers hide behind the GEMMs of the blocks that are already here.
    pipeline="blocking": one all_gather_into_tensor, then the GEMMs (the form measured first; kept for comparison).
    Kernels only ever read local memory: a peer's block is multiplied after it has landed in `recv`.
    """

    def __init__(self, kind: str, m: int, k: int, n_local: int, weight, world: int, device="cuda", activation: int = 0,
                 pipeline: str = "overlap", rank: int | None = None):
        from . import lib

        if kind not in ("w4a8", "nvfp4"):
            raise ValueError("ColumnSplitPlan: kind must be 'w4a8' or 'nvfp4'")
        if pipeline not in ("overlap", "blocking"):
            raise ValueError("ColumnSplitPlan: pipeline must be 'overlap' or 'blocking'")
        self.kind, self.m, self.k, self.n, self.world, self.weight, self.activation = kind, m, k, n_local, world, weight, activation
        self.pipeline = pipeline
        self.rank = rank if rank is not None else (dist.get_rank() if world > 1 else 0)
        if kind == "w4a8":
            self.q_bytes, self.s_bytes = m * k, 4 * m
        else:
            self.q_bytes, self.s_bytes = m * k // 2, lib.sfq_nvfp4_act_scale_bytes(m, k)
        self.q_bytes_padded = (self.q_bytes + 255) // 256 * 256
        self.block = self.q_bytes_padded + (self.s_bytes + 255) // 256 * 256
        self.send = torch.zeros(self.block, dtype=torch.uint8, device=device)
        self.recv = torch.zeros(world * self.block, dtype=torch.uint8, device=device)
        self.blocks = [self.recv[r * self.block:(r + 1) * self.block] for r in range(world)]
        self.y = torch.empty((world * m, n_local), dtype=torch.bfloat16, device=device)
        self.comm_stream = torch.cuda.Stream(device=device) if (world > 1 and pipeline == "overlap") else None
        self.ev_quantized = torch.cuda.Event() if self.comm_stream is not None else None
        self.ev_block = [torch.cuda.Event() for _ in range(world)] if self.comm_stream is not None else None
        self.gathered_bytes = self.block * (world - 1)

    def _quantize(self, x_local, q_ptr, s_ptr):
        from . import NVFP4_ACT_GEMM_FEED, check, lib, ptr, stream_ptr

        if self.kind == "w4a8":
            check(lib.sfq_quantize_int8_token(ptr(x_local), None, q_ptr, s_ptr, None, self.m, self.k, 1, stream_ptr()))
        else:
            check(lib.sfq_quantize_nvfp4_block(ptr(x_local), None, q_ptr, s_ptr, None, self.m, self.k, NVFP4_ACT_GEMM_FEED, stream_ptr()))

    def _gemm_block(self, base: int, r: int):
        import ctypes as C

        from . import F32, Epilogue, check, lib, ptr, stream_ptr

        m, k, n = self.m, self.k, self.n
        qb = base + r * self.block
        sb = qb + self.q_bytes_padded
        yb = ptr(self.y) + r * m * n * 2
        if self.kind == "w4a8":
            w8, col_scale = self.weight
            ep = Epilogue(sb, ptr(col_scale), 1.0, None, F32, self.activation)
            check(lib.sfq_gemm_int8(qb, ptr(w8), C.byref(ep), yb, m, n, k, stream_ptr()))
        else:
            data, scale, g = self.weight
            ep = Epilogue(None, None, g, None, F32, self.activation)
            check(lib.sfq_gemm_nvfp4(qb, sb, ptr(data), ptr(scale), C.byref(ep), yb, m, n, k, stream_ptr()))

    def gather_only(self, group=None) -> None:
        """The collective of forward() alone, on whatever the buffers hold (for timing it)."""
        if self.world == 1:
            return
        if self.pipeline == "blocking":
            dist.all_gather_into_tensor(self.recv, self.send, group=group)
        else:
            gather_blocks_stepwise(self.blocks, self.rank, group)

    def forward(self, x_local: torch.Tensor, group=None) -> torch.Tensor:
        """x_local bf16 [m, K] -> bf16 [world * m, n_local]: this rank's columns for all tokens."""
        from . import ptr

        if self.world == 1 or self.pipeline == "blocking":
            q_ptr = ptr(self.send)
            self._quantize(x_local, q_ptr, q_ptr + self.q_bytes_padded)
            if self.world > 1:
                dist.all_gather_into_tensor(self.recv, self.send, group=group)  # the one collective
                base = ptr(self.recv)
            else:
                base = ptr(self.send)
            for r in range(self.world):
                self._gemm_block(base, r)
            return self.y
        # ---- overlap: own block first, peers' blocks as they land
        compute = torch.cuda.current_stream()
        base = ptr(self.recv)
        q_ptr = base + self.rank * self.block
        self._quantize(x_local, q_ptr, q_ptr + self.q_bytes_padded)  # straight into this rank's slot of the gather
        self.ev_quantized.record(compute)  # also behind every GEMM of the previous call: their blocks may be overwritten
        self._gemm_block(base, self.rank)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(self.ev_quantized)
            gather_blocks_stepwise(self.blocks, self.rank, group, on_block=lambda src: self.ev_block[src].record(self.comm_stream))
        for _, src in exchange_steps(self.world, self.rank):
            compute.wait_event(self.ev_block[src])
            self._gemm_block(base, src)
        # the last event also covers this rank's last send: the next call may rewrite its slot
        return self.y
