"""Host side of the SpMM kernels: packed tile store, work plans and the launch itself.

Every function here ends in a call of the C ABI (include/void_b200.h).  Nothing computes on the
CPU; tensors that are not on a CUDA device are rejected.
"""
import ctypes
import weakref
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

TILE = 32
PANEL = 128
FLAG_DIRECT_STORES, FLAG_A_STABLE, FLAG_STORE_PER_TILE = 2, 4, 16   # bits of void_spmm_args.flags
FLAG_NO_EARLY_A = 1 << 30   # Python side only: never set FLAG_A_STABLE (measurements)


def _aligned_empty(nbytes: int, device, align: int = 1024) -> torch.Tensor:
    """uint8 buffer whose data pointer is ``align``-byte aligned."""
    raw = torch.empty(nbytes + align, dtype=torch.uint8, device=device)
    off = (-raw.data_ptr()) % align
    return raw[off:off + nbytes]


@dataclass
class PackedTiles:
    """A in the layout the kernels stream: tiles in tile-row-major order, 1024 elements each, already
    in the tensor cores' core-matrix order, with per-tile column index and scale."""
    tiles: torch.Tensor        # uint8 [nnz * 1024 * element bytes], 1024-byte aligned
    tile_cols: torch.Tensor    # int32 [nnz]
    tile_scales: torch.Tensor  # float32 [nnz]
    row_ptr: torch.Tensor      # int32 [nbr + 1]
    block_indices: torch.Tensor  # int32 [nnz]
    row_scale: torch.Tensor    # float32 [nbr]
    nbr: int
    nbc: int
    nnz: int
    shape: tuple
    kind: int                  # _lib.KIND_*
    terms: int = 1             # packed tiles per stored tile (2 / 3: FP8 tiles stored as sums of E4M3 terms)
    key: tuple = ()
    stable: bool = False       # the kernels that wrote the arrays above are known to have finished
    row_order: Optional[torch.Tensor] = None   # int32 [nbr]: tile rows by falling tile count (launches without a plan)

    def is_stable(self) -> bool:
        """True when no kernel still in flight can be writing this store.  A launch may then read
        the store before it waits for the previous kernel of its stream (flag bit 2 of void_spmm_args)."""
        return self.stable


def pack(values: torch.Tensor, scales: Optional[torch.Tensor], block_rows: torch.Tensor, block_cols: torch.Tensor,
         shape, kind: int, row_ptr=None, block_indices=None) -> PackedTiles:
    """Build the packed store of a VOID tensor on its device: void_pack_tiles for the 8-bit kinds,
    void_pack_tiles_fp for fp16 / bf16 / fp32 tiles (no scales)."""
    from .format import build_tile_index
    _lib.require_cuda(values, block_rows, block_cols)
    lib = _lib.load()
    dev = values.device
    M, K = shape
    nbr, nbc = (M + TILE - 1) // TILE, (K + TILE - 1) // TILE
    nnz = values.shape[0]
    es = _lib.KIND_ELEM_BYTES[kind]
    if values.dim() != 3 or values.shape[1] != TILE or values.shape[2] != TILE or values.element_size() != es:
        raise _lib.VoidB200Error("void_b200 kernels need 32x32 tiles of %d-byte elements here, got %s %s"
                                 % (es, tuple(values.shape), values.dtype))
    with torch.cuda.device(dev):
        if row_ptr is None or block_indices is None:
            row_ptr, block_indices = build_tile_index(block_rows, block_cols, nbr, nbc)
        vals = values.contiguous()
        tiles = _aligned_empty(max(nnz, 1) * 1024 * es, dev)
        tile_cols = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)
        tile_scales = torch.empty(max(nnz, 1), dtype=torch.float32, device=dev)
        row_scale = torch.empty(max(nbr, 1), dtype=torch.float32, device=dev)
        sc = None if scales is None else scales.contiguous().to(torch.float32).reshape(-1)
        bc = block_cols.contiguous().to(torch.int32)
        if es > 1:
            _lib.check(lib.void_pack_tiles_fp(_lib.ptr(vals), es, _lib.ptr(bc), _lib.ptr(block_indices), nnz,
                                              _lib.ptr(tiles), _lib.ptr(tile_cols), _lib.stream_ptr(dev)),
                       "void_pack_tiles_fp")
            return PackedTiles(tiles, tile_cols, tile_scales, row_ptr, block_indices, row_scale, nbr, nbc, nnz,
                               (M, K), kind)
        _lib.check(lib.void_pack_tiles(_lib.ptr(vals), _lib.ptr(sc), 0 if sc is None else sc.numel(), _lib.ptr(bc),
                                       _lib.ptr(block_indices), _lib.ptr(row_ptr), nnz, nbr, _lib.ptr(tiles),
                                       _lib.ptr(tile_cols), _lib.ptr(tile_scales), _lib.ptr(row_scale),
                                       _lib.stream_ptr(dev)), "void_pack_tiles")
    return PackedTiles(tiles, tile_cols, tile_scales, row_ptr, block_indices, row_scale, nbr, nbc, nnz,
                       (M, K), kind)


def pack_f8_split(values: torch.Tensor, scales: Optional[torch.Tensor], block_rows: torch.Tensor,
                  block_cols: torch.Tensor, shape, terms: int) -> PackedTiles:
    """Packed store of FP8 tiles with their scales folded in (void_pack_tiles_f8_split): every tile as a sum
    of ``terms`` E4M3 tiles relative to the largest tile scale of its tile row, which lands in row_scale."""
    from .format import build_tile_index
    _lib.require_cuda(values, block_rows, block_cols)
    lib = _lib.load()
    dev = values.device
    M, K = shape
    nbr, nbc = (M + TILE - 1) // TILE, (K + TILE - 1) // TILE
    nnz = values.shape[0]
    if values.dim() != 3 or tuple(values.shape[1:]) != (TILE, TILE) or values.element_size() != 1:
        raise _lib.VoidB200Error("void_b200 kernels need 32x32 FP8 tiles here, got %s %s" % (tuple(values.shape), values.dtype))
    with torch.cuda.device(dev):
        row_ptr, block_indices = build_tile_index(block_rows, block_cols, nbr, nbc)
        vals = values.contiguous()
        tiles = _aligned_empty(max(nnz, 1) * 1024 * terms, dev)
        tile_cols = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)
        tile_scales = torch.empty(max(nnz, 1), dtype=torch.float32, device=dev)
        row_scale = torch.empty(max(nbr, 1), dtype=torch.float32, device=dev)
        sc = None if scales is None else scales.contiguous().to(torch.float32).reshape(-1)
        br = block_rows.contiguous().to(torch.int32)
        bc = block_cols.contiguous().to(torch.int32)
        _lib.check(lib.void_pack_tiles_f8_split(_lib.ptr(vals), _lib.ptr(sc), 0 if sc is None else sc.numel(), _lib.ptr(br),
                                                _lib.ptr(bc), _lib.ptr(block_indices), _lib.ptr(row_ptr), nnz, nbr, terms,
                                                _lib.ptr(tiles), _lib.ptr(tile_cols), _lib.ptr(tile_scales),
                                                _lib.ptr(row_scale), _lib.stream_ptr(dev)), "void_pack_tiles_f8_split")
    return PackedTiles(tiles, tile_cols, tile_scales, row_ptr, block_indices, row_scale, nbr, nbc, nnz, (M, K),
                       _lib.KIND_F8E4M3, terms)


def _mark_ready(p: PackedTiles) -> PackedTiles:
    # Building a packed store is a one-time set-up step of a tensor (a weight): the host waits here until the
    # store is complete, so that every later launch may read it ahead of its stream order.  Inside a stream
    # capture nothing can be waited for; a store built there is simply never read early.
    # The CTAs that start first take the first work items: with the tile rows sorted by falling tile count the
    # longest rows start earliest and the shortest are left for the CTAs that share an SM with the most others.
    if p.nbr > 0:
        counts = p.row_ptr[1:] - p.row_ptr[:-1]
        p.row_order = torch.argsort(counts, descending=True, stable=True).to(torch.int32)
    if not torch.cuda.is_current_stream_capturing():
        torch.cuda.current_stream(p.tiles.device).synchronize()
        p.stable = True
    return p


def cached_pack(owner, values, scales, block_rows, block_cols, shape, kind) -> PackedTiles:
    """Packed store cached on the tensor object, rebuilt when its storage or contents change."""
    key = (kind, values.data_ptr(), values._version, None if scales is None else (scales.data_ptr(), scales._version),
           block_rows.data_ptr(), block_cols.data_ptr(), str(values.device), tuple(shape))
    p = getattr(owner, "_packed_cache", None)
    if p is None or p.key != key:
        p = _mark_ready(pack(values, scales, block_rows, block_cols, shape, kind))
        p.key = key
        owner._packed_cache = p
        owner._plan_cache = {}
    return p


_LIVE_PLANS = weakref.WeakSet()


def reset_plan_scratch(device) -> None:
    """Zero the split-row accumulators and counters of every live plan on ``device``.  A launch that gave up
    (status word set) may have left partial sums behind; the kernels only leave the scratch at zero when
    every split row was finished."""
    dev = torch.device(device)
    for plan in list(_LIVE_PLANS):
        if plan.counters.device == dev:
            plan.counters.zero_()
            if plan.partials is not None:
                plan.partials.zero_()


@dataclass(eq=False)
class Plan:
    """Work plan of void_plan_segments for one (packed tensor, column chunking, CTA count)."""
    segs: torch.Tensor
    cta_seg_ptr: torch.Tensor
    n_cta: int
    np: int
    n_chunks: int
    n_segs: int
    n_slots: int
    n_counters: int
    partials: Optional[torch.Tensor]
    counters: torch.Tensor
    mode: int
    chunk_tiles: int


def default_panels(nbr: int, N: int, sms: int) -> int:
    """Panels per work item the library picks by itself (same rule as the C launcher): two, unless
    that leaves fewer work items than four per SM."""
    panels = (N + PANEL - 1) // PANEL
    np_ = 2 if panels >= 2 else 1
    while np_ > 1 and nbr * ((panels + np_ - 1) // np_) < 4 * sms:
        np_ //= 2
    return np_


def sm_count(device) -> int:
    with torch.cuda.device(device):
        return _lib.load().void_device_sm_count()


def streamk_table(row_ptr: torch.Tensor, nbr: int, nnz: int, n_workers: Optional[int], max_work: int):
    """Worker table on the device (void_streamk_table).  Returns the four arrays trimmed to the
    realised worker count, the per-row worker offsets and the chunk length."""
    lib = _lib.load()
    dev = row_ptr.device
    req = -1 if n_workers is None else int(n_workers)
    if nnz == 0 or (n_workers is not None and req <= 0):
        raise ZeroDivisionError("integer division or modulo by zero")  # as void/stream_k.py:66
    target = lib.void_streamk_target(nnz, req, max_work)
    with torch.cuda.device(dev):
        cap = lib.void_streamk_table_capacity(nnz, nbr)
        rows = torch.empty(cap, dtype=torch.int32, device=dev)
        start = torch.empty(cap, dtype=torch.int32, device=dev)
        end = torch.empty(cap, dtype=torch.int32, device=dev)
        atomic = torch.empty(cap, dtype=torch.uint8, device=dev)
        n_out = torch.zeros(1, dtype=torch.int32, device=dev)
        woff = torch.empty(nbr + 1, dtype=torch.int32, device=dev)
        _lib.check(lib.void_streamk_table(_lib.ptr(row_ptr), nbr, nnz, req, max_work, _lib.ptr(rows), _lib.ptr(start),
                                          _lib.ptr(end), _lib.ptr(atomic), _lib.ptr(n_out), _lib.ptr(woff),
                                          _lib.stream_ptr(dev)), "void_streamk_table")
        n = int(n_out.item())
    return rows[:n], start[:n], end[:n], atomic[:n].to(torch.bool), woff, target


ROW_COST = 12  # epilogue of one (tile row, chunk) in units of one tile of work, swept on B200 (power-law workload: 6 -> 22.0 us, 12 -> 19.9, 24 -> 21.4)


def make_plan(packed: PackedTiles, N: int, np_: int, n_cta: int, mode: int, chunk_tiles: int = 0,
              woff: Optional[torch.Tensor] = None, row_cost: int = ROW_COST) -> Plan:
    """Cut the tile stream of ``packed`` into ``n_cta`` shares on the device (void_plan_segments)."""
    lib = _lib.load()
    dev = packed.row_ptr.device
    panels = (N + PANEL - 1) // PANEL
    n_chunks = (panels + np_ - 1) // np_
    with torch.cuda.device(dev):
        cap = lib.void_plan_capacity(packed.nnz, packed.nbr, n_chunks, n_cta, mode, chunk_tiles)
        segs = torch.empty(cap * 8, dtype=torch.int32, device=dev)
        cta_seg_ptr = torch.empty(n_cta + 1, dtype=torch.int32, device=dev)
        counts = torch.zeros(4, dtype=torch.int32, device=dev)
        ws_bytes = lib.void_plan_ws_bytes(packed.nbr, n_cta)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        _lib.check(lib.void_plan_segments(_lib.ptr(packed.row_ptr), packed.nbr, n_chunks, n_cta, mode, chunk_tiles,
                                          row_cost, _lib.ptr(woff), _lib.ptr(segs), cap, _lib.ptr(cta_seg_ptr), _lib.ptr(counts),
                                          _lib.ptr(ws), ws_bytes, _lib.stream_ptr(dev)), "void_plan_segments")
        n_segs, n_slots, n_ctr, overflow = (int(x) for x in counts.tolist())
        if overflow:
            raise _lib.VoidB200Error("void_plan_segments: segment list overflow")
        partials = None
        if n_ctr:   # one int32 accumulator per split row; the kernel leaves it zero again
            partials = torch.zeros(n_ctr * np_ * PANEL * TILE, dtype=torch.int32, device=dev)
        counters = torch.zeros(max(n_ctr, 1), dtype=torch.int32, device=dev)
    plan = Plan(segs, cta_seg_ptr, n_cta, np_, n_chunks, n_segs, n_slots, n_ctr, partials, counters, mode,
                chunk_tiles)
    _LIVE_PLANS.add(plan)
    return plan


def prepare_b(b: torch.Tensor, elem_bytes: int = 1) -> torch.Tensor:
    """B as the kernels need it: row-major, rows starting on 16-byte boundaries (the copy engine's rule)."""
    if b.element_size() != elem_bytes:
        raise _lib.VoidB200Error("B must have %d-byte elements to match A, got %s" % (elem_bytes, b.dtype))
    per16 = 16 // elem_bytes
    if b.stride(1) != 1 or b.stride(0) % per16 != 0 or b.data_ptr() % 16 != 0 or b.stride(0) < b.shape[1]:
        K, N = b.shape
        ld = (N + per16 - 1) // per16 * per16
        padded = torch.zeros(K, ld, dtype=b.dtype, device=b.device)
        padded[:, :N] = b
        b = padded[:, :N]
    return b


def spmm(packed: PackedTiles, b: torch.Tensor, out: torch.Tensor, *, scale_mode: int, col_scale=None,
         b_scale: float = 1.0, bias=None, act: int = 0, acc_out=None, plan: Optional[Plan] = None,
         worker_partials=None, use_row_scale: bool = True, panels_per_item: int = 0, stages: int = 0,
         grid: int = 0, tiles_per_stage: int = 0, cta_shape: int = 0, trace=None, flags: int = 0,
         row_bias=None, transposed: bool = False, test_hooks: int = 0, sorted_rows: Optional[bool] = None) -> torch.Tensor:
    """One launch of void_spmm_i8 / void_spmm_f8 / void_spmm_fp on the current stream of b's device.
    With ``transposed`` b is [N, K] and out is [N, M]: the product is out = b @ A^T, both used as they lie."""
    lib = _lib.load()
    _lib.require_cuda(b, out, packed.tiles)
    dev = b.device
    M, K = packed.shape
    N = b.shape[0] if transposed else b.shape[1]
    if (b.shape[1] if transposed else b.shape[0]) != K:
        raise _lib.VoidB200Error("shape mismatch: A is %s, B is %s" % (packed.shape, tuple(b.shape)))
    want = (N, M) if transposed else (M, N)
    if tuple(out.shape) != want or out.stride(1) != 1:
        raise _lib.VoidB200Error("out must be a row-major [%d, %d] tensor" % want)
    if out.dtype not in _lib.OUT_DTYPE_CODE:
        raise _lib.VoidB200Error("unsupported output dtype %s" % out.dtype)
    es = _lib.KIND_ELEM_BYTES[packed.kind]
    b = prepare_b(b, es)
    a = _lib.SpmmArgs()
    a.tiles = packed.tiles.data_ptr()
    a.tile_cols = packed.tile_cols.data_ptr()
    a.tile_scales = packed.tile_scales.data_ptr()
    a.row_ptr = packed.row_ptr.data_ptr()
    a.row_scale = packed.row_scale.data_ptr() if (use_row_scale and scale_mode == _lib.SCALE_ROW_MEAN and es == 1) else None
    a.nbr, a.nbc, a.nnz = packed.nbr, packed.nbc, packed.nnz
    a.b, a.ldb, a.K, a.N = b.data_ptr(), b.stride(0) * es, K, N
    keep = [b]
    if col_scale is not None:
        col_scale = col_scale.to(device=dev, dtype=torch.float32).contiguous()
        keep.append(col_scale)
        a.col_scale = col_scale.data_ptr()
    a.b_scale = float(b_scale)
    if bias is not None:
        bias = bias.to(device=dev, dtype=torch.float32).contiguous()
        keep.append(bias)
        a.bias = bias.data_ptr()
    if row_bias is not None:
        row_bias = row_bias.to(device=dev, dtype=torch.float32).contiguous()
        if row_bias.numel() != M:
            raise _lib.VoidB200Error("row bias must have %d elements, got %d" % (M, row_bias.numel()))
        keep.append(row_bias)
        a.row_bias = row_bias.data_ptr()
    a.out, a.ldc, a.M = out.data_ptr(), out.stride(0), M
    a.out_dtype = _lib.OUT_DTYPE_CODE[out.dtype]
    a.act = act
    a.scale_mode = scale_mode
    a.acc_out = None if acc_out is None else acc_out.data_ptr()
    if plan is not None:
        a.segs, a.cta_seg_ptr, a.n_cta = plan.segs.data_ptr(), plan.cta_seg_ptr.data_ptr(), plan.n_cta
        if plan.partials is not None:
            a.partials, a.partials_bytes = plan.partials.data_ptr(), plan.partials.numel() * 4
        a.counters = plan.counters.data_ptr()
        panels_per_item = plan.np
    # tile rows taken by falling tile count: measured on B200 at the 4096^2 sweep and at 16384^2, INT8 gains 3 - 5 %
    # (6.80 -> 6.58 us at 90 %, 10.33 -> 10.02 at 70 %, 72.7 -> 68.7 at 16384^2); FP8 tiles stored as two terms gain at
    # 90 % (7.88 -> 7.57) and lose at 70 % (13.55 -> 13.76), 16- and 32-bit tiles lose (TF32 70 %: 31.7 -> 33.1): the
    # balance it buys weighs less, and the scattered order of A more, the more bytes a tile row holds.  By default:
    # INT8 always, FP8 while a tile row averages at most 16 tiles, the floating kinds never
    if sorted_rows is None:
        sorted_rows = packed.kind == _lib.KIND_I8 or (packed.kind == _lib.KIND_F8E4M3 and packed.nnz <= 16 * packed.nbr)
    if plan is None and sorted_rows and packed.row_order is not None:
        a.row_order = packed.row_order.data_ptr()
    a.worker_partials = None if worker_partials is None else worker_partials.data_ptr()
    a.status = _lib.status_word(dev).data_ptr()
    a.panels_per_item, a.stages, a.grid, a.tiles_per_stage = panels_per_item, stages, grid, tiles_per_stage
    a.trace = None if trace is None else trace.data_ptr()
    a.cta_shape = cta_shape
    a.transposed = 1 if transposed else 0
    # bit 2: the packed store (and the plan, whose builder synchronises) is complete, so the kernel may
    # read it before it waits for the previous kernel of the stream
    a.flags = (flags & 0xffff) | (FLAG_A_STABLE if (packed.is_stable() and not (flags & FLAG_NO_EARLY_A)) else 0)
    a.test_hooks = test_hooks
    a.tile_terms = packed.terms
    with torch.cuda.device(dev):
        if es > 1:
            _lib.check(lib.void_spmm_fp(ctypes.byref(a), packed.kind, _lib.stream_ptr(dev)), "void_spmm_fp")
        else:
            fn = lib.void_spmm_i8 if packed.kind == _lib.KIND_I8 else lib.void_spmm_f8
            _lib.check(fn(ctypes.byref(a), _lib.stream_ptr(dev)), "void_spmm")
    return out
