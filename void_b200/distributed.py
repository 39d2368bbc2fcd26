"""ROW_WISE sharding of VOID tensors across the GPUs of one box, and the sharded SpMM.

Mirrors ShardingStrategy (void/distributed.py:10-14), DistributedVOIDTensor (:17-62),
shard_void_tensor (:84-196) and distributed_void_spmm (:199-270).

Each rank (one process per GPU) owns a contiguous range of tile rows,
rows_per_rank = ceil(n_block_rows / world_size) (:117-119), keeps those tiles in their original
(Morton) order with block_rows rebased to the range (:150-161) and multiplies them by a B that is
replicated on every GPU.  Tile rows are independent, so the product needs no collective: every
rank writes its own row shard of C.  B is replicated with one NCCL broadcast over NVLink
(broadcast_b) - the reference expects B to be there already.  The reference's all_gather of the
full C onto every rank (:234-250) is available as gather_output=True (the default, to keep the
reference's return value); gather_output=False returns the local row shard.

The reference's shard_void_tensor raises TypeError (its VOIDTensor(...) call omits required
fields, :179-186); this one fills them in and also accepts Int8VOIDTensor / FP8VOIDTensor.

COLUMN_WISE (:127-137) and BLOCK_WISE (:139-145) give every rank tiles of ALL tile rows, so the
per-rank products are partial sums of the whole C and the reference adds them with an all_reduce of
the full [M, N] matrix (:252-267).  Here the sum is part of the INT8 SpMM kernel itself
(fused_reduce_spmm): output tile rows are owned by ranks (the ROW_WISE ranges), every rank adds its
int32 partial tiles straight into the owner's accumulator through peer memory (NVLink), bumps the
owner's arrival counter, and whichever rank arrives last reads the finished sums back, dequantises
and writes the owner's rows of C - a reduce-scatter without a separate collective and without any
kernel waiting for another GPU.  Integer adds commute, so the result does not depend on arrival order.

nnz-balanced ROW_WISE ranges (balance="nnz") cut the tile rows where the running tile count crosses
k/world of the total instead of at equal row counts; the reference's ranges stay the default.
"""
from dataclasses import dataclass
from enum import Enum
from typing import Optional, Tuple, Union

import torch
import torch.distributed as dist

from .format import VOIDTensor
from .fp8 import FP8ScalingInfo, FP8VOIDTensor, void_spmm_fp8
from .int_quant import Int8VOIDTensor, void_spmm_int8


class ShardingStrategy(Enum):
    ROW_WISE = "row_wise"
    COLUMN_WISE = "column_wise"
    BLOCK_WISE = "block_wise"


@dataclass
class DistributedVOIDTensor:
    """Local shard plus sharding metadata (void/distributed.py:17-62).  The fields after
    local_col_range are additions: row_ranges lists every rank's tile-row range when it is not the
    reference's equal split (balance="nnz"); global_row_scale carries the mean tile scale of every
    tile row of the WHOLE tensor, which the INT8 epilogue needs when a rank holds only part of a row."""
    local_tensor: Union[VOIDTensor, Int8VOIDTensor, FP8VOIDTensor]
    strategy: ShardingStrategy
    world_size: int
    rank: int
    global_shape: Tuple[int, int]
    local_row_range: Tuple[int, int]
    local_col_range: Tuple[int, int]
    row_ranges: Optional[Tuple[Tuple[int, int], ...]] = None
    global_row_scale: Optional[torch.Tensor] = None

    @property
    def device(self) -> torch.device:
        return self.local_tensor.block_rows.device

    @property
    def n_local_blocks(self) -> int:
        return self.local_tensor.n_blocks

    def to(self, device) -> "DistributedVOIDTensor":
        return DistributedVOIDTensor(self.local_tensor.to(device), self.strategy, self.world_size, self.rank,
                                     self.global_shape, self.local_row_range, self.local_col_range, self.row_ranges,
                                     None if self.global_row_scale is None else self.global_row_scale.to(device))

    def owner_ranges(self) -> Tuple[Tuple[int, int], ...]:
        """Tile rows [start, end) of C each rank owns: this tensor's row ranges for ROW_WISE, the
        reference's equal split of the rows for the strategies that reduce."""
        if self.row_ranges is not None:
            return self.row_ranges
        tile_m = self.local_tensor.tile_size[0]
        nbr = (self.global_shape[0] + tile_m - 1) // tile_m
        return tuple(row_range(nbr, self.world_size, r) for r in range(self.world_size))


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size() -> int:
    return dist.get_world_size() if is_distributed() else 1


def get_rank() -> int:
    return dist.get_rank() if is_distributed() else 0


def row_range(n_block_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Tile rows [start, end) of a rank (void/distributed.py:117-119)."""
    rows_per_rank = (n_block_rows + world_size - 1) // world_size
    start = min(rank * rows_per_rank, n_block_rows)
    return start, min(start + rows_per_rank, n_block_rows)


def balanced_row_ranges(block_rows: torch.Tensor, n_block_rows: int, world_size: int) -> Tuple[Tuple[int, int], ...]:
    """Contiguous tile-row ranges that minimise the largest number of stored tiles any rank gets (the
    bottleneck partition: binary search on the capacity, greedy fill).  Equal row counts (the reference's
    split) leave ranks idle when the tiles per row are far from uniform."""
    counts = torch.bincount(block_rows.to(torch.int64).cpu(), minlength=n_block_rows)[:n_block_rows].tolist()

    def cuts_for(capacity):
        cuts, load = [0], 0
        for r, c in enumerate(counts):
            if load + c > capacity and load > 0:
                cuts.append(r)
                load = 0
            load += c
        return cuts

    lo, hi = max(counts + [0]), max(sum(counts), 1)
    while lo < hi:
        mid = (lo + hi) // 2
        if len(cuts_for(mid)) <= world_size:
            hi = mid
        else:
            lo = mid + 1
    cuts = cuts_for(lo)
    cuts += [n_block_rows] * (world_size + 1 - len(cuts))      # ranks past the last cut own nothing
    return tuple((cuts[k], cuts[k + 1]) for k in range(world_size))


def _take(void_tensor, indices, local_rows, local_cols, local_shape, grid_cells):
    """The tiles ``indices`` of a VOIDTensor / Int8VOIDTensor / FP8VOIDTensor as a tensor of the same class."""
    n_local = int(indices.numel())
    tile_m, tile_k = void_tensor.tile_size
    if isinstance(void_tensor, Int8VOIDTensor):
        return Int8VOIDTensor(values=void_tensor.values[indices], scales=void_tensor.scales[indices],
                              zero_points=void_tensor.zero_points[indices], block_rows=local_rows,
                              block_cols=local_cols, shape=local_shape, tile_size=void_tensor.tile_size,
                              n_blocks=n_local, config=void_tensor.config)
    if isinstance(void_tensor, FP8VOIDTensor):
        s = void_tensor.scaling_info
        per_tile = s.scale.dim() == 1 and s.scale.numel() == void_tensor.n_blocks
        pick = (lambda t: t[indices]) if per_tile else (lambda t: t)
        info = FP8ScalingInfo(scale=pick(s.scale), scale_inv=pick(s.scale_inv), amax=pick(s.amax),
                              amax_history=pick(s.amax_history), config=s.config)
        return FP8VOIDTensor(values_fp8=void_tensor.values_fp8[indices], scaling_info=info, block_rows=local_rows,
                             block_cols=local_cols, morton_codes=void_tensor.morton_codes[indices], shape=local_shape,
                             tile_size=void_tensor.tile_size, nnz_original=n_local * tile_m * tile_k,
                             n_blocks=n_local, density=n_local / grid_cells)
    values = void_tensor.values[indices]
    return VOIDTensor(values=values, block_rows=local_rows, block_cols=local_cols,
                      morton_codes=void_tensor.morton_codes[indices], shape=local_shape,
                      tile_size=void_tensor.tile_size,
                      nnz_original=int(torch.count_nonzero(values).item()) if n_local else 0,
                      n_blocks=n_local, density=n_local / grid_cells, dtype=void_tensor.dtype)


def shard_void_tensor(void_tensor, strategy: ShardingStrategy = ShardingStrategy.ROW_WISE,
                      world_size: Optional[int] = None, rank: Optional[int] = None, *,
                      balance: str = "rows") -> DistributedVOIDTensor:
    """Keep this rank's tiles of a VOIDTensor / Int8VOIDTensor / FP8VOIDTensor (void/distributed.py:84-196).

    ROW_WISE: tile rows [rank * ceil(nbr / world), ...) with block_rows rebased (:115-125, :159-161);
    balance="nnz" replaces the equal split by balanced_row_ranges.  COLUMN_WISE: block columns
    [rank * ceil(nbc / world), ...), block_cols NOT rebased, local shape shrunk to the range
    (:127-137, :173-176).  BLOCK_WISE: stored tile i goes to rank i % world (:139-145).
    Kept tiles stay in their stored (Morton) order.
    """
    if world_size is None:
        world_size = get_world_size()
    if rank is None:
        rank = get_rank()
    if not isinstance(strategy, ShardingStrategy):
        raise ValueError(f"Unknown sharding strategy: {strategy}")
    if balance not in ("rows", "nnz"):
        raise ValueError("balance must be 'rows' or 'nnz'")
    n_block_rows, n_block_cols = void_tensor.block_grid
    tile_m, tile_k = void_tensor.tile_size
    row_ranges = None
    global_row_scale = None
    if strategy == ShardingStrategy.ROW_WISE:
        if balance == "nnz":
            row_ranges = balanced_row_ranges(void_tensor.block_rows, n_block_rows, world_size)
            start_row, end_row = row_ranges[rank]
        else:
            start_row, end_row = row_range(n_block_rows, world_size, rank)
        mask = (void_tensor.block_rows >= start_row) & (void_tensor.block_rows < end_row)
        local_row_range, local_col_range = (start_row, end_row), (0, n_block_cols)
        local_shape = ((end_row - start_row) * tile_m, void_tensor.shape[1])
    elif strategy == ShardingStrategy.COLUMN_WISE:
        cols_per_rank = (n_block_cols + world_size - 1) // world_size
        start_col = min(rank * cols_per_rank, n_block_cols)
        end_col = min(start_col + cols_per_rank, n_block_cols)
        mask = (void_tensor.block_cols >= start_col) & (void_tensor.block_cols < end_col)
        local_row_range, local_col_range = (0, n_block_rows), (start_col, end_col)
        local_shape = (void_tensor.shape[0], (end_col - start_col) * tile_k)
    else:
        positions = torch.arange(void_tensor.n_blocks, device=void_tensor.block_rows.device)
        mask = (positions % world_size) == rank
        local_row_range, local_col_range = (0, n_block_rows), (0, n_block_cols)
        local_shape = tuple(void_tensor.shape)
    indices = torch.where(mask)[0]
    local_rows = void_tensor.block_rows[indices].to(torch.int32)
    if strategy == ShardingStrategy.ROW_WISE:
        local_rows = (void_tensor.block_rows[indices] - local_row_range[0]).to(torch.int32)
    local_cols = void_tensor.block_cols[indices]
    cells = max((local_row_range[1] - local_row_range[0]) * (local_col_range[1] - local_col_range[0]), 1)
    local = _take(void_tensor, indices, local_rows, local_cols, local_shape, cells)
    if strategy != ShardingStrategy.ROW_WISE and isinstance(void_tensor, Int8VOIDTensor) and void_tensor.values.is_cuda:
        # INT8 semantic: a tile row's accumulator is scaled by the mean of ALL of the row's tile scales
        # (void/int_quant.py:516-526); a rank that holds part of the row needs the whole row's mean
        global_row_scale = void_tensor.packed().row_scale[:n_block_rows].clone()
    return DistributedVOIDTensor(local_tensor=local, strategy=strategy, world_size=world_size, rank=rank,
                                 global_shape=tuple(void_tensor.shape), local_row_range=local_row_range,
                                 local_col_range=local_col_range, row_ranges=row_ranges,
                                 global_row_scale=global_row_scale)


def broadcast_b(b: torch.Tensor, src: int = 0, group=None, scales: Optional[torch.Tensor] = None):
    """Replicate B (and its per-column scales) from rank ``src`` on every rank: one broadcast of
    the 8-bit matrix over NCCL / NVLink, issued once at set-up."""
    if is_distributed() and get_world_size() > 1:
        # collectives move plain bytes: view float8 as uint8
        payload = b.view(torch.uint8) if b.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else b
        dist.broadcast(payload, src=src, group=group)
        if scales is not None:
            dist.broadcast(scales, src=src, group=group)
    return b, scales


def _local_spmm(local, b, b_scale, out_dtype, out=None):
    if isinstance(local, Int8VOIDTensor):
        return void_spmm_int8(local, b, b_scale, out, out_dtype=out_dtype)
    if isinstance(local, FP8VOIDTensor):
        return void_spmm_fp8(local, b, out_dtype or torch.float16, b_scale=b_scale, out=out)
    if isinstance(local, VOIDTensor):
        from .ops import void_spmm
        res = void_spmm(local, b, out)
        return res if out_dtype in (None, res.dtype) else res.to(out_dtype)
    raise NotImplementedError("distributed_void_spmm takes shards of VOIDTensor, Int8VOIDTensor or FP8VOIDTensor")


def broadcast_spmm_overlapped(dist_tensor: DistributedVOIDTensor, b: torch.Tensor, scales: Optional[torch.Tensor] = None,
                              *, src: int = 0, panel_cols: int = 256, out: Optional[torch.Tensor] = None,
                              out_dtype: Optional[torch.dtype] = None, group=None):
    """The first product after B has been produced on rank ``src``: B travels in panels of ``panel_cols``
    columns, and every rank multiplies a panel while the next one is still on the wire.

    On entry ``b`` [K, N] (and ``scales`` [N]) hold data on rank ``src`` and are receive buffers of the same
    shape elsewhere; on return every rank holds all of B, like after broadcast_b, and the local row shard of
    C = A @ B is returned.  Panels are staged in contiguous [K, panel] buffers (a collective moves
    contiguous bytes), broadcast on a side stream, multiplied on the current stream as they arrive
    (the kernel takes the panel as its B and writes the matching columns of the row shard) and copied
    into ``b``.  No kernel waits on another GPU: the order is kept by stream events on each rank.
    """
    local = dist_tensor.local_tensor
    K, N = b.shape
    rows = local.shape[0]
    if out is None:
        out = torch.empty(rows, N, dtype=out_dtype or torch.float32, device=b.device)
    multi = is_distributed() and get_world_size() > 1
    rank = get_rank() if multi else src
    payload = b.view(torch.uint8) if b.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else b
    if multi and scales is not None:
        dist.broadcast(scales, src=src, group=group)
    on_gpu = b.is_cuda
    main = torch.cuda.current_stream(b.device) if on_gpu else None
    side = _side_stream(b.device) if (on_gpu and multi) else None
    if side is not None:
        side.wait_stream(main)                         # B's producer ran on the current stream
    staged = []
    for c0 in range(0, N, panel_cols):
        c1 = min(c0 + panel_cols, N)
        ready = None
        if multi:
            ctx = torch.cuda.stream(side) if side is not None else _NullContext()
            with ctx:
                panel = torch.empty(K, c1 - c0, dtype=payload.dtype, device=b.device)
                if rank == src:
                    panel.copy_(payload[:, c0:c1])
                dist.broadcast(panel, src=src, group=group)
                if side is not None:
                    ready = torch.cuda.Event()
                    ready.record(side)
            staged.append(panel)                       # stays alive until the streams are joined below
            if ready is not None:
                main.wait_event(ready)
            if rank != src:
                payload[:, c0:c1].copy_(panel)
            panel_b = panel.view(b.dtype)
        else:
            panel_b = b[:, c0:c1]
        sc = None if scales is None else scales[c0:c1]
        _local_spmm(local, panel_b, sc, out.dtype, out[:, c0:c1])
    if side is not None:
        side.wait_stream(main)                         # the panels may be freed once the products have run
    return out, b


_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    """One communication stream per device, kept between calls: the caching allocator hands a freed staging
    buffer back only to the stream it was allocated on, so a fresh stream per call would allocate anew each time."""
    key = torch.device(device).index
    st = _SIDE_STREAMS.get(key)
    if st is None:
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return st


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _gather_rows(shard: torch.Tensor, ranges, rank: int, M: int, tile_m: int, out: Optional[torch.Tensor]) -> torch.Tensor:
    """all_gather of row shards of unequal height (padded to the tallest) into the full [M, N] result."""
    N = shard.shape[1]
    rows_max = max(e - s for s, e in ranges) * tile_m
    padded = torch.zeros(rows_max, N, dtype=shard.dtype, device=shard.device)
    padded[:shard.shape[0]] = shard
    gathered = [torch.empty_like(padded) for _ in ranges]
    dist.all_gather(gathered, padded)
    if out is None:
        out = torch.empty(M, N, dtype=shard.dtype, device=shard.device)
    for (s, e), g in zip(ranges, gathered):
        start, end = s * tile_m, min(e * tile_m, M)
        if end > start:
            out[start:end] = g[:end - start]
    return out


def distributed_void_spmm(dist_tensor: DistributedVOIDTensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
                          async_op: bool = False, *, b_scale=None, out_dtype: Optional[torch.dtype] = None,
                          gather_output: bool = True) -> torch.Tensor:
    """C = A @ B with A sharded over the ranks (void/distributed.py:199-270).

    b must be replicated on every rank (see broadcast_b).
    ROW_WISE: every rank multiplies its tile rows; with gather_output=True the full [M, N] result is returned
    on every rank like the reference does (:234-250), with gather_output=False each rank returns its own row
    shard [(end - start) * tile_m, N] and no collective runs.
    COLUMN_WISE / BLOCK_WISE: the per-rank products are partial sums of all of C (:252-267).  For Int8 shards on
    GPUs the sum happens inside the kernel (reduce.fused_reduce_spmm: every rank ends up with the finished rows
    it owns, which gather_output=True then gathers); other tensors take the reference's route, a local product
    followed by dist.all_reduce of the full result.
    """
    import dataclasses
    M, K = dist_tensor.global_shape
    local = dist_tensor.local_tensor
    tile_m = local.tile_size[0]
    ranges = dist_tensor.owner_ranges()
    if dist_tensor.strategy != ShardingStrategy.ROW_WISE:
        whole = dataclasses.replace(local, shape=(M, K)) if tuple(local.shape) != (M, K) else local
        if dist_tensor.world_size == 1:
            return _local_spmm(whole, b, b_scale, out_dtype, out)
        if isinstance(local, Int8VOIDTensor) and b.is_cuda and dist_tensor.global_row_scale is not None:
            from .reduce import fused_reduce_spmm
            shard = fused_reduce_spmm(dist_tensor, b, b_scale, out_dtype)
            if not gather_output:
                return shard
            return _gather_rows(shard, ranges, dist_tensor.rank, M, tile_m, out)
        if isinstance(local, Int8VOIDTensor):
            raise NotImplementedError("Int8 shards by column or block need the whole rows' mean scales: shard on the GPU")
        partial = _local_spmm(whole, b, b_scale, torch.float32)
        dist.all_reduce(partial, op=dist.ReduceOp.SUM)
        res = partial if out_dtype in (None, torch.float32) else partial.to(out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    local_out = _local_spmm(local, b, b_scale, out_dtype, out if not gather_output else None)
    if dist_tensor.world_size == 1 or not gather_output:
        return local_out[:M] if dist_tensor.world_size == 1 else local_out
    return _gather_rows(local_out, ranges, dist_tensor.rank, M, tile_m, out)


__all__ = ["ShardingStrategy", "DistributedVOIDTensor", "shard_void_tensor", "distributed_void_spmm", "broadcast_b",
           "broadcast_spmm_overlapped",
           "row_range", "is_distributed", "get_world_size", "get_rank"]
