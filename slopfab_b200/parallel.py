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


def row_chunks(rows: int, chunks: int, multiple: int = 128) -> list[tuple[int, int]]:
    """(first row, row count) of at most `chunks` contiguous pieces of `rows` rows; every piece starts on a multiple of
    `multiple` rows (128 keeps the fp4 scale tiles of a piece whole), the last one takes the ragged end."""
    if rows < 0 or chunks <= 0 or multiple <= 0:
        raise ValueError("row_chunks: bad arguments")
    units = (rows + multiple - 1) // multiple
    pieces = []
    for c in range(min(chunks, max(units, 1))):
        u0, uc = token_shard(units, min(chunks, max(units, 1)), c)
        r0, r1 = u0 * multiple, min(rows, (u0 + uc) * multiple)
        if r1 > r0:
            pieces.append((r0, r1 - r0))
    return pieces


class ColumnSplitPlan:
    """FFN-up column split with preallocated buffers and equal token counts per rank (the benchmark's case).

    Every rank quantizes its own `m` token rows into blocks [quantized rows | their scales]; the blocks of all ranks are
    brought into ordinary local memory by NCCL all-gather (the one collective of the scheme) and the local weight columns
    are multiplied block by block, one GEMM launch per source rank and row chunk, so no block waits for a repack. Kinds:
    "w4a8" (int8 rows + fp32 row scales; `weight` = (int8 [n_local, K], col_scale fp32 [n_local])) and "nvfp4" (fp4
    rows + 128x4-tiled e4m3 scales; `weight` = (u8 [n_local, K/2], tiled scales, global_scale)).

    pipeline="overlap" (default): the rows are cut into `chunks` pieces (128-row aligned). The rank's own pieces are
      multiplied at once, straight from the send buffers, while a communication stream gathers piece after piece; one
      event per gathered piece releases the GEMMs of the peers' rows of that piece, so the later pieces travel behind
      the GEMMs of the earlier ones.
    pipeline="blocking": one all_gather_into_tensor of everything, then the GEMMs.
    Kernels only ever read local memory: a peer's rows are multiplied after they have landed in `recv`.
    """

    def __init__(self, kind: str, m: int, k: int, n_local: int, weight, world: int, device="cuda", activation: int = 0,
                 pipeline: str = "overlap", rank: int | None = None, chunks: int = 2):
        from . import lib

        if kind not in ("w4a8", "nvfp4"):
            raise ValueError("ColumnSplitPlan: kind must be 'w4a8' or 'nvfp4'")
        if pipeline not in ("overlap", "blocking"):
            raise ValueError("ColumnSplitPlan: pipeline must be 'overlap' or 'blocking'")
        self.kind, self.m, self.k, self.n, self.world, self.weight, self.activation = kind, m, k, n_local, world, weight, activation
        self.pipeline = pipeline
        self.rank = rank if rank is not None else (dist.get_rank() if world > 1 else 0)
        self.pieces = row_chunks(m, chunks if (pipeline == "overlap" and world > 1) else 1)
        pad = lambda b: (b + 255) // 256 * 256  # noqa: E731
        self.q_pad, self.sub = [], []
        for _, rows in self.pieces:
            q = rows * k if kind == "w4a8" else rows * k // 2
            sc = 4 * rows if kind == "w4a8" else lib.sfq_nvfp4_act_scale_bytes(rows, k)
            self.q_pad.append(pad(q))
            self.sub.append(pad(q) + pad(sc))
        self.send = [torch.zeros(b, dtype=torch.uint8, device=device) for b in self.sub]
        self.recv = [torch.zeros(world * b, dtype=torch.uint8, device=device) for b in self.sub]
        self.y = torch.empty((world * m, n_local), dtype=torch.bfloat16, device=device)
        overlap = world > 1 and pipeline == "overlap"
        self.comm_stream = torch.cuda.Stream(device=device) if overlap else None
        self.ev_quantized = torch.cuda.Event() if overlap else None
        self.ev_piece = [torch.cuda.Event() for _ in self.pieces] if overlap else None
        self.gathered_bytes = sum(self.sub) * (world - 1)

    def _quantize(self, x_local, c):
        from . import NVFP4_ACT_GEMM_FEED, check, lib, ptr, stream_ptr

        r0, rows = self.pieces[c]
        x_ptr = ptr(x_local) + r0 * self.k * 2
        q_ptr = ptr(self.send[c])
        s_ptr = q_ptr + self.q_pad[c]
        if self.kind == "w4a8":
            check(lib.sfq_quantize_int8_token(x_ptr, None, q_ptr, s_ptr, None, rows, self.k, 1, stream_ptr()))
        else:
            check(lib.sfq_quantize_nvfp4_block(x_ptr, None, q_ptr, s_ptr, None, rows, self.k, NVFP4_ACT_GEMM_FEED, stream_ptr()))

    def _gemm(self, qb: int, c: int, src: int):
        """y[rows of piece c of source rank src, :] from the quantized block at device address qb."""
        import ctypes as C

        from . import F32, Epilogue, check, lib, ptr, stream_ptr

        r0, rows = self.pieces[c]
        k, n = self.k, self.n
        sb = qb + self.q_pad[c]
        yb = ptr(self.y) + (src * self.m + r0) * n * 2
        if self.kind == "w4a8":
            w8, col_scale = self.weight
            ep = Epilogue(sb, ptr(col_scale), 1.0, None, F32, self.activation)
            check(lib.sfq_gemm_int8(qb, ptr(w8), C.byref(ep), yb, rows, n, k, stream_ptr()))
        else:
            data, scale, g = self.weight
            ep = Epilogue(None, None, g, None, F32, self.activation)
            check(lib.sfq_gemm_nvfp4(qb, sb, ptr(data), ptr(scale), C.byref(ep), yb, rows, n, k, stream_ptr()))

    def gather_only(self, group=None) -> None:
        """The collective of forward() alone, on whatever the buffers hold (for timing it)."""
        if self.world == 1:
            return
        for c in range(len(self.pieces)):
            dist.all_gather_into_tensor(self.recv[c], self.send[c], group=group)

    def forward(self, x_local: torch.Tensor, group=None) -> torch.Tensor:
        """x_local bf16 [m, K] -> bf16 [world * m, n_local]: this rank's columns for all tokens."""
        from . import ptr

        pieces = range(len(self.pieces))
        for c in pieces:
            self._quantize(x_local, c)
        if self.world == 1:
            for c in pieces:
                self._gemm(ptr(self.send[c]), c, 0)
            return self.y
        if self.pipeline == "blocking":
            for c in pieces:
                dist.all_gather_into_tensor(self.recv[c], self.send[c], group=group)  # the one collective (one piece)
            for src in range(self.world):
                for c in pieces:
                    self._gemm(ptr(self.recv[c]) + src * self.sub[c], c, src)
            return self.y
        # ---- overlap: own rows first, the peers' rows piece by piece as they land
        compute = torch.cuda.current_stream()
        self.ev_quantized.record(compute)  # also behind every GEMM of the previous call: their blocks may be overwritten
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(self.ev_quantized)
            for c in pieces:
                dist.all_gather_into_tensor(self.recv[c], self.send[c], group=group)
                self.ev_piece[c].record(self.comm_stream)
        for c in pieces:
            self._gemm(ptr(self.send[c]), c, self.rank)
        for c in pieces:
            compute.wait_event(self.ev_piece[c])  # the last one also says the send buffers may be rewritten
            for src in range(self.world):
                if src != self.rank:
                    self._gemm(ptr(self.recv[c]) + src * self.sub[c], c, src)
        return self.y
