"""Stream-K load balancing for power-law tile-row lengths on B200.

Mirrors StreamKWorkload (void/stream_k.py:13-33), compute_stream_k_workload (:36-110),
void_spmm_stream_k (:233-301) and analyze_workload_balance (:467-492).

The worker table is the reference's, bit for bit, but it is built by a device kernel instead of a
Python loop with one .item() per row (:76-97).  The SpMM differs in how partial rows are joined:
the reference lets every partial worker lock the output tile and read-modify-write it in the
output dtype (:198-219, an unbounded spin); here consecutive workers of a row that land on the
same CTA keep accumulating in tensor memory, rows that are shared between CTAs add their partial
sums into one accumulator per row with atomic adds, and the CTA that arrives last reads it back
and runs the epilogue - no lock and no wait.  For an Int8VOIDTensor the sums are int32, exact and
independent of arrival order; for a floating VOIDTensor (the reference's own argument type) they
are fp32 and their last bits depend on the order, as the reference's locked adds do.
"""
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, _spmm
from .format import VOIDTensor
from .int_quant import Int8VOIDTensor, _resolve_b


@dataclass
class StreamKWorkload:
    """Per-worker assignments (void/stream_k.py:13-33)."""
    worker_rows: torch.Tensor          # [n_workers] int32
    worker_block_start: torch.Tensor   # [n_workers] int32
    worker_block_end: torch.Tensor     # [n_workers] int32
    worker_needs_atomic: torch.Tensor  # [n_workers] bool
    n_workers: int
    total_work: int
    # extras used by the B200 launch (not part of the reference dataclass)
    chunk_tiles: int = 0
    worker_offsets: Optional[torch.Tensor] = None


def compute_stream_k_workload(void_tensor, n_workers: Optional[int] = None,
                              max_work_per_worker: int = 16) -> StreamKWorkload:
    """Stream-K work distribution (void/stream_k.py:36-110): rows in order, every non-empty row cut
    into chunks of target = min(ceil(n_blocks / n_workers), max_work_per_worker) tiles."""
    row_ptr, _ = void_tensor.get_row_block_info()
    nbr = void_tensor.block_grid[0]
    rows, start, end, atomic, woff, target = _spmm.streamk_table(row_ptr, nbr, void_tensor.n_blocks, n_workers,
                                                                  max_work_per_worker)
    return StreamKWorkload(worker_rows=rows, worker_block_start=start, worker_block_end=end,
                           worker_needs_atomic=atomic, n_workers=rows.numel(), total_work=void_tensor.n_blocks,
                           chunk_tiles=target, worker_offsets=woff)


def _plan_for(a, packed, N: int, workload: StreamKWorkload, per_worker: bool, n_cta: Optional[int]):
    sms = _spmm.sm_count(packed.tiles.device)
    np_ = _spmm.default_panels(packed.nbr, N, sms) if _lib.KIND_ELEM_BYTES[packed.kind] == 1 else 1
    if n_cta is None:
        n_cta = sms * 4          # four slim CTAs per SM
    mode = 2 if per_worker else 1
    key = ("streamk", packed.kind, N, np_, n_cta, mode, workload.chunk_tiles)
    cache = getattr(a, "_plan_cache", None)
    if cache is None:
        cache = a._plan_cache = {}
    plan = cache.get(key)
    if plan is None:
        plan = _spmm.make_plan(packed, N, np_, n_cta, mode, workload.chunk_tiles, workload.worker_offsets)
        cache[key] = plan
    return plan


def void_spmm_stream_k(a: Int8VOIDTensor, b: torch.Tensor, workload: Optional[StreamKWorkload] = None,
                       out: Optional[torch.Tensor] = None, *, b_scale=None, out_dtype: Optional[torch.dtype] = None,
                       activation: int = 0, bias: Optional[torch.Tensor] = None,
                       worker_partials: Optional[torch.Tensor] = None, acc_out: Optional[torch.Tensor] = None,
                       n_cta: Optional[int] = None) -> torch.Tensor:
    """Load-balanced SpMM (void/stream_k.py:233-301): a floating VOIDTensor as in the reference, or an
    Int8VOIDTensor with the fused epilogue of void_spmm_int8 (``b_scale`` / ``out_dtype`` apply to it).

    ``worker_partials`` (int32 [n_segments, 32, N], see the plan's segment list) makes every worker of
    the table a segment of its own and records its partial sum - the check that the sum of the
    partials is the row accumulator.
    """
    assert b.dim() == 2
    assert a.shape[1] == b.shape[0]
    _lib.require_cuda(a.values, b)
    if isinstance(a, VOIDTensor):
        return _stream_k_fp(a, b, workload, out, activation, bias, worker_partials, acc_out, n_cta)
    if not isinstance(a, Int8VOIDTensor):
        raise TypeError("void_spmm_stream_k takes a VOIDTensor or an Int8VOIDTensor, got %s" % type(a).__name__)
    M, K = a.shape
    N = b.shape[1]
    b_q, scalar, col_scale = _resolve_b(b, b_scale)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.float32, device=b.device)
    packed = a.packed()
    if a.n_blocks == 0:
        return _spmm.spmm(packed, b_q, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=col_scale, b_scale=scalar,
                          bias=bias, act=activation)
    if workload is None:
        workload = _cached_workload(a)
    plan = _plan_for(a, packed, N, workload, worker_partials is not None, n_cta)
    return _spmm.spmm(packed, b_q, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=col_scale, b_scale=scalar, bias=bias,
                      act=activation, plan=plan, worker_partials=worker_partials, acc_out=acc_out)


def _cached_workload(a) -> StreamKWorkload:
    """The table depends on A's structure only: built once per tensor, then reused."""
    workload = getattr(a, "_streamk_workload_cache", None)
    if workload is None or workload.total_work != a.n_blocks:
        workload = compute_stream_k_workload(a)
        a._streamk_workload_cache = workload
    return workload


def _stream_k_fp(a: VOIDTensor, b, workload, out, activation, bias, worker_partials, acc_out, n_cta):
    """void_spmm_stream_k on a floating VOIDTensor (void/stream_k.py:233-301): result in B's dtype."""
    from . import ops
    if a.n_blocks == 0:
        return ops.void_spmm(a, b, out, activation=activation, bias=bias)
    if workload is None:
        workload = _cached_workload(a)
    packed = ops.packed_fp(a, ops.product_kind(a, b))
    plan = _plan_for(a, packed, b.shape[1], workload, worker_partials is not None, n_cta)
    return ops.void_spmm(a, b, out, activation=activation, bias=bias, plan=plan, acc_out=acc_out,
                         worker_partials=worker_partials)


def stream_k_plan(a, N: int, workload: StreamKWorkload, per_worker: bool = False, n_cta: Optional[int] = None,
                  kind: Optional[int] = None) -> _spmm.Plan:
    """The device-built work plan void_spmm_stream_k uses for an N-column product (``kind``: the
    product kind of a floating VOIDTensor, fp32 operands by default)."""
    if isinstance(a, VOIDTensor):
        from . import ops
        packed = ops.packed_fp(a, _lib.FP_KIND.get(a.values.dtype, _lib.KIND_TF32) if kind is None else kind)
    else:
        packed = a.packed()
    return _plan_for(a, packed, N, workload, per_worker, n_cta)


def analyze_workload_balance(void_tensor) -> dict:
    """Row-length statistics (void/stream_k.py:467-492)."""
    row_ptr, _ = void_tensor.get_row_block_info()
    row_work = (row_ptr[1:] - row_ptr[:-1]).float()
    non_empty = row_work > 0
    nz = row_work[non_empty]
    if len(nz) == 0:
        return {"empty": True}
    return {
        "empty": False,
        "n_rows": len(row_work),
        "n_nonempty_rows": non_empty.sum().item(),
        "min_blocks_per_row": nz.min().item(),
        "max_blocks_per_row": nz.max().item(),
        "mean_blocks_per_row": nz.mean().item(),
        "std_blocks_per_row": nz.std().item(),
        "imbalance_ratio": (nz.max() / nz.mean()).item(),
        "coefficient_of_variation": (nz.std() / nz.mean()).item(),
    }


__all__ = ["StreamKWorkload", "compute_stream_k_workload", "void_spmm_stream_k", "analyze_workload_balance",
           "stream_k_plan"]
