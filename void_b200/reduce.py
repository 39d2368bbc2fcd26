"""INT8 SpMM whose sum over ranks happens inside the kernel: the product of COLUMN_WISE / BLOCK_WISE shards.

The reference multiplies every rank's shard by B and adds the full [M, N] results with dist.all_reduce
(void/distributed.py:252-267).  Here every (tile row, column chunk) of C has an OWNER rank (the ROW_WISE
ranges).  Each rank runs the row-accumulate kernel over all tile rows with a plan whose segments name the
owner; the kernel adds its int32 partial tile into the owner's accumulator through peer memory
(system-scope atomic adds, NVLink), bumps the owner's arrival counter, and the rank that arrives last
reads the sums back, dequantises and writes the owner's rows of C.  That is a reduce-scatter without a
collective in the data path, and no kernel waits for another GPU.  Integer adds commute, so the result
is the one-GPU result bit for bit.

Two forms of it are built (``mode`` of fused_reduce_spmm):
  "slots" (default)  every rank STORES its int32 partial tile into its own slot of the owner's scratch (plain
                     16 KB tiles over NVLink at copy speed, no atomics, no counters); after the ordering
                     all_reduce the owner adds the slots of its rows and dequantises (void_reduce_slots, a
                     bandwidth-bound pass over local memory).  Slots are double-buffered by call parity, so one
                     all_reduce per call orders everything.
  "atomic"           the single-kernel form described above (system-scope atomic adds, last arriver finishes);
                     needs world times less scratch, but 4-byte atomic adds over NVLink run at a quarter of the
                     copy bandwidth.

Scratch (per rank: int32 accumulators for the rows it owns, their counters, its rows of C) lives in one
buffer that every rank can address: torch's symmetric memory when it can be set up, else CUDA IPC handles
of an ordinary allocation.  Consecutive launches are ordered by one small all_reduce on the stream: it ends
only when every rank's kernel has finished, which is also when a rank's rows of C are complete.
"""
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib, _spmm

TILE, PANEL = _spmm.TILE, _spmm.PANEL
MAX_PEERS = 8


def reduce_segments(row_ptr: torch.Tensor, n_chunks: int, world_size: int, rank: int,
                    owner_ranges: Sequence[Tuple[int, int]], n_cta: int):
    """Plan of the reducing launch of one rank: one segment per (tile row, column chunk) of the WHOLE matrix,
    8 int32 each as void_plan_segments writes them: (row, chunk, first tile, end tile, contributors = world
    size, owner rank, this rank, index of the row's accumulator in the owner's scratch).  The list starts
    with the rows of the rank after this one, so that the ranks do not all push to the same owner at once,
    and is cut into n_cta runs of (nearly) equal length.  Plain tensor arithmetic: runs on CPU tensors too."""
    dev = row_ptr.device
    nbr = row_ptr.numel() - 1
    rows = torch.arange(nbr, device=dev, dtype=torch.int64)
    owner = torch.zeros(nbr, dtype=torch.int64, device=dev)
    start_of = torch.zeros(nbr, dtype=torch.int64, device=dev)
    for r, (s, e) in enumerate(owner_ranges):
        if e > s:
            owner[s:e] = r
            start_of[s:e] = s
    first = owner_ranges[(rank + 1) % world_size][0] if world_size > 1 else 0
    order = torch.roll(rows, -int(first))                         # rows in the order this rank visits them
    row_i = order.repeat_interleave(n_chunks)
    chunk_i = torch.arange(n_chunks, device=dev, dtype=torch.int64).repeat(nbr)
    rp = row_ptr.to(torch.int64)
    segs = torch.stack([row_i, chunk_i, rp[row_i], rp[row_i + 1], torch.full_like(row_i, world_size), owner[row_i],
                        torch.full_like(row_i, rank), (row_i - start_of[row_i]) * n_chunks + chunk_i], dim=1)
    n_items = nbr * n_chunks
    n_cta = max(1, min(n_cta, n_items))
    cta_seg_ptr = (torch.arange(n_cta + 1, device=dev, dtype=torch.int64) * n_items) // n_cta
    return segs.to(torch.int32).contiguous(), cta_seg_ptr.to(torch.int32).contiguous(), n_cta


@dataclass
class Scratch:
    """One rank's part of the shared scratch and everybody's addresses of it."""
    buffer: torch.Tensor                 # uint8, this rank's buffer
    ptrs: List[int]                      # base address of every rank's buffer as seen from this GPU
    acc_bytes: int                       # accumulators of the owned rows
    ctr_off: int
    out_off: int
    keep: object = None                  # whatever must stay alive for the peer mappings
    slots: bool = False                  # slot form: acc_bytes is the size of ONE of the two slot sets


def _layout(rows_max: int, n_chunks: int, np_: int, N: int, out_bytes: int, slot_ranks: int = 0):
    """Offsets inside a rank's scratch.  Atomic form: accumulators, counters, the rank's rows of C.  Slot form
    (slot_ranks = world size): two sets of per-rank slots, nothing else."""
    if slot_ranks:
        one = rows_max * n_chunks * slot_ranks * np_ * PANEL * TILE * 4
        return one, 2 * one, 2 * one, 2 * one
    acc = rows_max * n_chunks * np_ * PANEL * TILE * 4
    ctr_off = (acc + 255) // 256 * 256
    out_off = (ctr_off + rows_max * n_chunks * 4 + 255) // 256 * 256
    total = out_off + rows_max * TILE * N * out_bytes
    return acc, ctr_off, out_off, (total + 255) // 256 * 256


def shared_buffer(nbytes: int, device, group=None) -> Tuple[torch.Tensor, List[int], object]:
    """A zeroed buffer of ``nbytes`` on every rank of ``group`` plus, on each rank, the addresses under which
    this GPU reaches every rank's buffer.  All ranks must call it with the same size.
    First choice is torch's symmetric memory (without an NVLink multicast binding: nothing here uses multimem);
    if that cannot be set up, an ordinary allocation is shared through CUDA IPC handles."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    dev = torch.device(device)
    if world == 1:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        return buf, [buf.data_ptr()], None
    err = None
    ok = torch.zeros(1, dtype=torch.int32, device=dev)
    buf = hdl = None
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        hdl = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        off = buf.data_ptr() - ptrs[rank]
        ptrs = [p + off for p in ptrs]
        ok.fill_(1)
    except Exception as ex:          # noqa: BLE001 - any failure selects the IPC route, on every rank
        err = ex
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 1:
        buf.zero_()
        return buf, ptrs, hdl
    # CUDA IPC: every rank exports its allocation, opens the others'
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    handle = buf.untyped_storage()._share_cuda_()
    handles = [None] * world
    dist.all_gather_object(handles, handle, group=group)
    peers, ptrs = [], []
    for r in range(world):
        if r == rank:
            ptrs.append(buf.data_ptr())
            continue
        h = list(handles[r])
        h[0] = dev.index if dev.index is not None else torch.cuda.current_device()   # map it on THIS device
        st = torch.UntypedStorage._new_shared_cuda(*h)
        t = torch.empty(0, dtype=torch.uint8, device=dev).set_(st)
        peers.append(t)
        ptrs.append(t.data_ptr())
    return buf, ptrs, (peers, err)


@dataclass
class ReduceState:
    """Everything the reducing launch of one sharded tensor needs, built once and cached on the tensor."""
    packed: _spmm.PackedTiles
    segs: torch.Tensor
    cta_seg_ptr: torch.Tensor
    n_cta: int
    np: int
    n_chunks: int
    N: int
    out_dtype: torch.dtype
    ranges: Tuple[Tuple[int, int], ...]
    scratch: Scratch
    token: torch.Tensor                  # the word the ordering all_reduce adds up
    contrib: Optional[torch.Tensor] = None    # slot form: uint8 per owned tile row, bit r = rank r holds tiles of the row
    out: Optional[torch.Tensor] = None        # slot form: this rank's rows of C (ordinary memory)
    calls: int = 0                            # slot form: parity selects the slot set


def launch_reduce(state: ReduceState, b: torch.Tensor, col_scale: Optional[torch.Tensor], b_scalar: float,
                  scratch_ptrs: Sequence[int], rank_count: int, act: int = 0, bias=None, slot_set: int = 0) -> None:
    """One reducing launch on the current stream: void_spmm_i8 with n_peers = rank_count and, per owner rank,
    the addresses of its accumulators, counters and rows of C inside the buffer ``scratch_ptrs[owner]``."""
    import ctypes
    lib = _lib.load()
    pk = state.packed
    dev = b.device
    M, K = pk.shape
    b = _spmm.prepare_b(b, 1)
    a = _lib.SpmmArgs()
    a.tiles, a.tile_cols, a.tile_scales = pk.tiles.data_ptr(), pk.tile_cols.data_ptr(), pk.tile_scales.data_ptr()
    a.row_ptr, a.row_scale = pk.row_ptr.data_ptr(), pk.row_scale.data_ptr()
    a.nbr, a.nbc, a.nnz = pk.nbr, pk.nbc, pk.nnz
    a.b, a.ldb, a.K, a.N = b.data_ptr(), b.stride(0), K, state.N
    keep = [b]
    if col_scale is not None:
        col_scale = col_scale.to(device=dev, dtype=torch.float32).contiguous()
        keep.append(col_scale)
        a.col_scale = col_scale.data_ptr()
    if bias is not None:
        bias = bias.to(device=dev, dtype=torch.float32).contiguous()
        keep.append(bias)
        a.bias = bias.data_ptr()
    a.b_scale = float(b_scalar)
    sc = state.scratch
    elem = torch.empty(0, dtype=state.out_dtype).element_size()
    a.out, a.ldc, a.M = scratch_ptrs[0] + sc.out_off, state.N, M     # a.out only has to be non-null here
    a.out_dtype, a.act, a.scale_mode = _lib.OUT_DTYPE_CODE[state.out_dtype], act, _lib.SCALE_ROW_MEAN
    a.segs, a.cta_seg_ptr, a.n_cta = state.segs.data_ptr(), state.cta_seg_ptr.data_ptr(), state.n_cta
    a.partials_bytes = sc.acc_bytes
    a.status = _lib.status_word(dev).data_ptr()
    a.panels_per_item = state.np
    a.flags = _spmm.FLAG_A_STABLE if pk.is_stable() else 0
    a.n_peers = rank_count
    a.peer_slots = 1 if sc.slots else 0
    for r in range(rank_count):
        base = scratch_ptrs[r] + (slot_set * sc.acc_bytes if sc.slots else 0)
        a.peer_partials[r] = base
        a.peer_counters[r] = base + sc.ctr_off
        # the owner's rows of C, moved back by its first row so that the global tile row indexes it
        a.peer_out[r] = base + sc.out_off - state.ranges[r][0] * TILE * state.N * elem
    with torch.cuda.device(dev):
        _lib.check(lib.void_spmm_i8(ctypes.byref(a), _lib.stream_ptr(dev)), "void_spmm_i8 (reduce)")


def contributors(row_ptr: torch.Tensor, rank: int, group=None) -> torch.Tensor:
    """uint8 per tile row of the whole matrix: bit r set when rank r holds at least one tile of the row
    (every rank knows its own rows; the masks are added up over the ranks - the bits are distinct)."""
    mine = ((row_ptr[1:] - row_ptr[:-1]) > 0).to(torch.int32) << rank
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(mine, group=group)
    return mine.to(torch.uint8)


def build_state(dist_tensor, N: int, out_dtype: torch.dtype, group=None, n_cta: Optional[int] = None,
                scratch: Optional[Scratch] = None, mode: str = "slots") -> ReduceState:
    """Pack the local tiles against the GLOBAL shape, build the plan and (unless given) the shared scratch."""
    from .int_quant import Int8VOIDTensor
    local = dist_tensor.local_tensor
    if not isinstance(local, Int8VOIDTensor):
        raise NotImplementedError("the reducing SpMM is built for Int8VOIDTensor shards (integer sums commute)")
    if dist_tensor.world_size > MAX_PEERS:
        raise ValueError("at most %d ranks" % MAX_PEERS)
    if mode not in ("slots", "atomic"):
        raise ValueError("mode must be 'slots' or 'atomic'")
    if dist_tensor.global_row_scale is None:
        raise ValueError("shard the tensor with shard_void_tensor on its CUDA device: the mean tile scale of whole rows is needed")
    dev = local.values.device
    M, K = dist_tensor.global_shape
    world, rank = dist_tensor.world_size, dist_tensor.rank
    packed = _spmm.pack(local.values, local.scales, local.block_rows, local.block_cols, (M, K), _lib.KIND_I8)
    packed.row_scale = dist_tensor.global_row_scale.to(device=dev, dtype=torch.float32).contiguous()
    sms = _spmm.sm_count(dev)
    panels = (N + PANEL - 1) // PANEL
    np_ = 2 if panels >= 2 else 1
    n_chunks = (panels + np_ - 1) // np_
    ranges = tuple(dist_tensor.owner_ranges())
    segs, cta_seg_ptr, n_cta = reduce_segments(packed.row_ptr, n_chunks, world, rank, ranges, n_cta or 4 * sms)
    packed = _spmm._mark_ready(packed)     # the host waits here: the store AND the plan are complete before any launch reads them early
    rows_max = max(e - s for s, e in ranges)
    elem = torch.empty(0, dtype=out_dtype).element_size()
    slots = mode == "slots" and world > 1      # a single rank has nothing to add up: its rows are finished in the launch
    acc, ctr_off, out_off, total = _layout(rows_max, n_chunks, np_, N, elem, world if slots else 0)
    made_here = scratch is None
    if made_here:
        buf, ptrs, keep = shared_buffer(total, dev, group)
        scratch = Scratch(buf, ptrs, acc, ctr_off, out_off, keep, slots)
    contrib = out = None
    if slots and made_here:
        s0, e0 = ranges[rank]
        contrib = contributors(packed.row_ptr, rank, group)[s0:e0].contiguous()
        out = torch.empty(max(e0 - s0, 0) * TILE, N, dtype=out_dtype, device=dev)
    if made_here:
        torch.cuda.synchronize(dev)                      # zeroed everywhere before anybody writes into it
        if dist.is_initialized() and world > 1:
            dist.barrier(group)
    token = torch.zeros(1, dtype=torch.int32, device=dev)
    return ReduceState(packed, segs, cta_seg_ptr, n_cta, np_, n_chunks, N, out_dtype, ranges, scratch, token, contrib, out)


def reduce_owned_rows(state: ReduceState, slots_ptr: int, contrib: torch.Tensor, rank: int, world: int, col_scale, b_scalar: float,
                      out: torch.Tensor, act: int = 0, bias=None) -> torch.Tensor:
    """Slot form, second half: add the per-rank partial tiles of this rank's rows (void_reduce_slots)."""
    lib = _lib.load()
    dev = out.device
    s0, e0 = state.ranges[rank]
    M = state.packed.shape[0]
    panels = (state.N + PANEL - 1) // PANEL
    keep = []
    if col_scale is not None:
        col_scale = col_scale.to(device=dev, dtype=torch.float32).contiguous()
        keep.append(col_scale)
    if bias is not None:
        bias = bias.to(device=dev, dtype=torch.float32).contiguous()
        keep.append(bias)
    import ctypes
    with torch.cuda.device(dev):
        _lib.check(lib.void_reduce_slots(ctypes.c_void_p(slots_ptr), _lib.ptr(contrib), world, max(e0 - s0, 0), s0, panels, state.np,
                                         _lib.ptr(state.packed.row_scale), _lib.ptr(col_scale), float(b_scalar), _lib.ptr(bias), act,
                                         _lib.ptr(out), out.stride(0) if out.numel() else state.N, _lib.OUT_DTYPE_CODE[out.dtype], M, state.N,
                                         _lib.stream_ptr(dev)), "void_reduce_slots")
    return out


def fused_reduce_spmm(dist_tensor, b: torch.Tensor, b_scale=None, out_dtype: Optional[torch.dtype] = None,
                      group=None, activation: int = 0, bias=None, mode: str = "slots") -> torch.Tensor:
    """This rank's rows of C = A @ B for an Int8 tensor sharded COLUMN_WISE or BLOCK_WISE: [(end - start) * 32, N]
    for the rank's range of DistributedVOIDTensor.owner_ranges().  The returned tensor belongs to the sharded
    tensor's state: it is overwritten by the next call on it.  Every rank must make the same calls."""
    from .int_quant import _resolve_b
    out_dtype = out_dtype or torch.float32
    N = b.shape[1]
    b_q, scalar, col_scale = _resolve_b(b, b_scale)
    key = (N, out_dtype, mode)
    cache = dist_tensor.__dict__.setdefault("_reduce_states", {})
    st = cache.get(key)
    if st is None:
        st = cache[key] = build_state(dist_tensor, N, out_dtype, group, mode=mode)
    world, rank = dist_tensor.world_size, dist_tensor.rank
    multi = dist.is_initialized() and world > 1
    sc = st.scratch
    if sc.slots:
        which = st.calls & 1
        st.calls += 1
        # activation and bias belong to the finished sums: the SpMM launches only store raw partial tiles
        launch_reduce(st, b_q, None, 1.0, sc.ptrs, world, 0, None, slot_set=which)
        if multi:
            dist.all_reduce(st.token, group=group)       # ends when every rank's launch has ended: the slots are complete
        reduce_owned_rows(st, sc.ptrs[rank] + which * sc.acc_bytes, st.contrib, rank, world, col_scale, scalar, st.out,
                          activation, bias)
        s, e = st.ranges[rank]
        return st.out[:max(min(e * TILE, dist_tensor.global_shape[0]) - s * TILE, 0)]
    launch_reduce(st, b_q, col_scale, scalar, sc.ptrs, world, activation, bias)
    if multi:
        # ends when every rank's kernel has ended: this rank's rows are complete, and the scratch may be used again
        dist.all_reduce(st.token, group=group)
    s, e = st.ranges[rank]
    rows = min(e * TILE, dist_tensor.global_shape[0]) - s * TILE if e > s else 0
    elem = torch.empty(0, dtype=out_dtype).element_size()
    return sc.buffer[sc.out_off: sc.out_off + max(rows, 0) * N * elem].view(out_dtype).view(max(rows, 0), N)
