"""CPU restatement of the reference's quantized block-sparse SpMM path (numpy / torch-CPU).

TEST INFRASTRUCTURE ONLY.  This module is the checker of the CUDA path: only the tests, the
smoke check and the benchmark's CPU-baseline leg import it.  Nothing in the ``void_b200``
package imports, calls or falls back to it.

Every function restates one piece of Khushiyant/void and cites the file:line it follows.
Pinning: the functions are checked in tests/test_oracle_golden.py against fixtures under
tests/golden/ that were produced by running the reference itself (its Triton kernels on the
CPU interpreter) through tests/golden/make_golden.py.  Two pieces have no reference run to pin
them, because the reference code raises before returning (its VOIDTensor constructor calls
miss required fields): the ROW_WISE sharding arithmetic (void/distributed.py:115-172) —
"parity unpinned" for that function — everything else is pinned.
"""
import numpy as np
import torch

TILE = 32


# ----------------------------------------------------------------------------- format
def morton_encode_batch(rows, cols):
    """16 bits per axis interleaved, rows on even bits: void/format.py:41-51."""
    def spread(v):
        v = np.asarray(v).astype(np.uint64)
        v = (v | (v << np.uint64(8))) & np.uint64(0x00FF00FF)
        v = (v | (v << np.uint64(4))) & np.uint64(0x0F0F0F0F)
        v = (v | (v << np.uint64(2))) & np.uint64(0x33333333)
        v = (v | (v << np.uint64(1))) & np.uint64(0x55555555)
        return v
    return spread(rows) | (spread(cols) << np.uint64(1))


def csr_to_void_fields(matrix, tile_size=TILE):
    """Vectorised restatement of csr_to_void, void/format.py:278-349.

    Active blocks = blocks holding at least one STORED entry (explicit zeros count, :287-296),
    sorted by Morton code (:305-311); duplicates inside a block: last write wins (:321-327).
    """
    coo = matrix.tocoo()
    M, N = matrix.shape
    rows, cols, data = coo.row.astype(np.int64), coo.col.astype(np.int64), coo.data
    nbr = (M + tile_size - 1) // tile_size
    nbc = (N + tile_size - 1) // tile_size
    keys = (rows // tile_size) * nbc + (cols // tile_size)
    uniq, inverse = np.unique(keys, return_inverse=True)
    n_blocks = len(uniq)
    brow, bcol = uniq // nbc, uniq % nbc
    morton = morton_encode_batch(brow, bcol)
    order = np.argsort(morton)
    reverse = np.zeros(n_blocks, dtype=np.int64)
    reverse[order] = np.arange(n_blocks)
    values = np.zeros((n_blocks, tile_size, tile_size), dtype=np.float32)
    values[reverse[inverse], rows % tile_size, cols % tile_size] = data
    return {
        "values": values,
        "block_rows": brow[order].astype(np.int32),
        "block_cols": bcol[order].astype(np.int32),
        "morton_codes": morton[order].astype(np.int64),
        "shape": (M, N),
        "n_blocks": n_blocks,
        "nnz_original": int(matrix.nnz),
        "density": n_blocks / (nbr * nbc),
    }


def dense_to_void_fields(matrix, threshold=0.0, tile_size=TILE):
    """dense_to_void, void/format.py:352-446: zero-pad to whole tiles (:374-378), keep the tiles whose sum of
    |x| exceeds the threshold (:391-394), order them by Morton code (:413-424); nnz_original counts the
    nonzero elements of the unpadded matrix (:429)."""
    a = np.asarray(matrix)
    M, N = a.shape
    nbr, nbc = (M + tile_size - 1) // tile_size, (N + tile_size - 1) // tile_size
    padded = np.zeros((nbr * tile_size, nbc * tile_size), dtype=a.dtype)
    padded[:M, :N] = a
    tiles = padded.reshape(nbr, tile_size, nbc, tile_size).transpose(0, 2, 1, 3)
    norms = np.abs(tiles).sum(axis=(2, 3))
    rows, cols = np.nonzero(norms > threshold)
    codes = morton_encode_batch(rows, cols)
    order = np.argsort(codes)
    n = len(rows)
    return {
        "values": tiles[rows[order], cols[order]] if n else np.zeros((0, tile_size, tile_size), a.dtype),
        "block_rows": rows[order].astype(np.int32), "block_cols": cols[order].astype(np.int32),
        "morton_codes": codes[order].astype(np.int64), "shape": (M, N), "n_blocks": n,
        "nnz_original": int(np.count_nonzero(a)), "density": (n / (nbr * nbc)) if n else 0.0,
    }


def row_block_info(block_rows, block_cols, nbr, nbc):
    """row_ptr and block_indices of VOIDTensor.get_row_block_info, void/format.py:218-231."""
    block_rows = np.asarray(block_rows, dtype=np.int64)
    block_cols = np.asarray(block_cols, dtype=np.int64)
    counts = np.bincount(block_rows, minlength=nbr)
    row_ptr = np.zeros(nbr + 1, dtype=np.int32)
    row_ptr[1:] = np.cumsum(counts)
    block_indices = np.argsort(block_rows * nbc + block_cols, kind="stable").astype(np.int32)
    return row_ptr, block_indices


# ----------------------------------------------------------------------------- INT8 quantisation
def quantize_int8_tiles(values):
    """Per-block symmetric INT8: quantize_void_tensor -> quantize_tensor -> compute_scale_minmax,
    void/int_quant.py:363-369, :286-294, :201-212.  scale = max(|min|,|max|)/128 clamped to 1e-8,
    q = round_half_even(x / scale) clamped to [-128, 127]."""
    v = torch.as_tensor(values, dtype=torch.float32)
    flat = v.reshape(v.shape[0], -1)
    absmax = torch.maximum(flat.amin(dim=1).abs(), flat.amax(dim=1).abs())
    scale = torch.clamp(absmax / 128, min=1e-8)
    q = (v / scale[:, None, None]).round().clamp(-128, 127).to(torch.int8)
    return q.numpy(), scale.numpy()


def quantize_int8_cols(b):
    """Per-column INT8 of a [K, N] matrix: the reference API on the transpose,
    quantize_tensor(B.T, PER_CHANNEL), void/int_quant.py:273-274, :194-212, :288."""
    bt = torch.as_tensor(b, dtype=torch.float32).t().contiguous()
    absmax = torch.maximum(bt.amin(dim=1, keepdim=True).abs(), bt.amax(dim=1, keepdim=True).abs())
    scale = torch.clamp(absmax / 128, min=1e-8)
    q = (bt / scale).round().clamp(-128, 127).to(torch.int8)
    return q.t().contiguous().numpy(), scale.reshape(-1).numpy()


# ----------------------------------------------------------------------------- FP8 quantisation
def _fp8_scale(amax):
    # FP8ScalingInfo.compute_scale with a fresh history, void/fp8.py:91-105 (margin 0)
    scale = torch.clamp(amax / 448.0, min=1e-12)
    return scale, 1.0 / scale


def quantize_fp8_tiles(values):
    """Per-block E4M3: quantize_to_fp8(scale_mode='per_block'), void/fp8.py:185-229, :159-182.
    Returns (bytes uint8, scale, scale_inv, amax)."""
    v = torch.as_tensor(values, dtype=torch.float32)
    amax = v.reshape(v.shape[0], -1).abs().max(dim=1).values
    scale, scale_inv = _fp8_scale(amax)
    scaled = torch.clamp(v * scale_inv.view(-1, 1, 1), -448.0, 448.0)
    q = scaled.to(torch.float8_e4m3fn)
    return q.view(torch.uint8).numpy(), scale.numpy(), scale_inv.numpy(), amax.numpy()


def quantize_fp8_cols(b):
    """Per-column E4M3 of a [K, N] matrix: quantize_to_fp8(B.T, scale_mode='per_row'),
    void/fp8.py:177-180, :217-227."""
    bt = torch.as_tensor(b, dtype=torch.float32).t().contiguous()
    amax = bt.abs().max(dim=1).values
    scale, scale_inv = _fp8_scale(amax)
    q = torch.clamp(bt * scale_inv.view(-1, 1), -448.0, 448.0).to(torch.float8_e4m3fn)
    return q.t().contiguous().view(torch.uint8).numpy(), scale.numpy(), scale_inv.numpy()


def fp8_bytes_to_float(q):
    return torch.as_tensor(np.ascontiguousarray(q)).view(torch.float8_e4m3fn).float().numpy()


# ----------------------------------------------------------------------------- SpMM
def _row_order(block_rows, block_cols, shape):
    M, K = shape
    nbr, nbc = (M + TILE - 1) // TILE, (K + TILE - 1) // TILE
    row_ptr, bidx = row_block_info(block_rows, block_cols, nbr, nbc)
    return nbr, nbc, row_ptr, bidx


def _b_block(b, c, K):
    """Rows [32c, 32c+32) of B, zero-padded past K (boundary_check of the block pointer,
    void/int_quant.py:504-512)."""
    blk = b[c * TILE:min((c + 1) * TILE, K)]
    if blk.shape[0] < TILE:
        blk = np.concatenate([blk, np.zeros((TILE - blk.shape[0], b.shape[1]), dtype=b.dtype)])
    return blk


def spmm_fp(values, block_rows, block_cols, shape, b, t_range=None):
    """fp32 result of void_spmm_kernel, void/ops.py:93-146: for every tile of the row, in row order,
    acc += float32(A tile) @ float32(B block) with an fp32 accumulator (on a GPU tl.dot rounds the
    operands to TF32, so a device result agrees to about 1e-3, the bar of tests/test_all_features.py:48).
    With t_range=(t0, t1) only the tiles at row-ordered positions [t0, t1) are added (one Stream-K
    worker, void/stream_k.py:166-193).  ``values`` [nnz, 32, 32] and ``b`` [K, N] are cast to fp32."""
    nbr, nbc, row_ptr, bidx = _row_order(block_rows, block_cols, shape)
    M, K = shape
    N = b.shape[1]
    a = np.asarray(values, dtype=np.float32)
    bf = np.asarray(b, dtype=np.float32)
    out = np.zeros((nbr * TILE, N), dtype=np.float32)
    for r in range(nbr):
        lo, hi = int(row_ptr[r]), int(row_ptr[r + 1])
        if t_range is not None:
            lo, hi = max(lo, t_range[0]), min(hi, t_range[1])
        acc = np.zeros((TILE, N), dtype=np.float32)
        for i in bidx[lo:hi]:
            acc = acc + np.matmul(a[i], _b_block(bf, int(block_cols[i]), K))
        out[r * TILE:(r + 1) * TILE] = acc
    return out[:M]


def spmm_int8_acc(values_q, block_rows, block_cols, shape, b_q, t_range=None):
    """int32 accumulators acc[nbr*32, N] = sum over the row's tiles of A_q . B_q, the tl.dot of
    void/int_quant.py:484-516.  float64 BLAS is exact here (|sum| < 2^53).  With t_range=(t0, t1)
    only the tiles at row-ordered positions [t0, t1) are added (one Stream-K worker,
    void/stream_k.py:166-193)."""
    nbr, nbc, row_ptr, bidx = _row_order(block_rows, block_cols, shape)
    K = shape[1]
    N = b_q.shape[1]
    bq = np.asarray(b_q).astype(np.float64)
    acc = np.zeros((nbr * TILE, N), dtype=np.float64)
    for r in range(nbr):
        lo, hi = int(row_ptr[r]), int(row_ptr[r + 1])
        if t_range is not None:
            lo, hi = max(lo, t_range[0]), min(hi, t_range[1])
        if hi <= lo:
            continue
        idx = bidx[lo:hi]
        a_cat = np.concatenate([values_q[i].astype(np.float64) for i in idx], axis=1)
        b_cat = np.concatenate([_b_block(bq, int(block_cols[i]), K) for i in idx], axis=0)
        acc[r * TILE:(r + 1) * TILE] = a_cat @ b_cat
    return acc.astype(np.int64).astype(np.int32)


def int8_row_scale(scales, block_rows, block_cols, shape, b_scale=1.0):
    """avg_scale of each tile row: fp32 running sum of a_scale * b_scale in row order, divided by
    the tile count, void/int_quant.py:518-526.  Empty rows get 0."""
    nbr, nbc, row_ptr, bidx = _row_order(block_rows, block_cols, shape)
    out = np.zeros(nbr, dtype=np.float32)
    bs = np.float32(b_scale)
    for r in range(nbr):
        lo, hi = int(row_ptr[r]), int(row_ptr[r + 1])
        if hi == lo:
            continue
        s = np.float32(0.0)
        for i in bidx[lo:hi]:
            s = np.float32(s + np.float32(np.float32(scales[i]) * bs))
        out[r] = np.float32(s / np.float32(hi - lo))
    return out


def spmm_int8(values_q, scales, block_rows, block_cols, shape, b_q, b_scale=1.0, col_scale=None):
    """fp32 result of void_spmm_int8, void/int_quant.py:523-540: float(acc) * mean row scale.
    Per-column scales of B (an extension; the reference result is linear in b_scale) multiply the
    b_scale = 1 result column by column."""
    M = shape[0]
    acc = spmm_int8_acc(values_q, block_rows, block_cols, shape, b_q)
    rs = int8_row_scale(scales, block_rows, block_cols, shape, b_scale)
    out = acc.astype(np.float32) * np.repeat(rs, TILE)[:, None]
    if col_scale is not None:
        out = out * np.asarray(col_scale, dtype=np.float32)[None, :]
    return out[:M].astype(np.float32)


_C_LIB = None


def c_library():
    """The compiled C restatement (oracle/void_oracle_c.c), built on first use; None without a C compiler."""
    global _C_LIB
    if _C_LIB is None:
        import ctypes
        from . import build_c
        try:
            path = build_c.build()
            _C_LIB = ctypes.CDLL(path) if path else False
        except (OSError, RuntimeError):
            _C_LIB = False
        if _C_LIB:
            vp, i32, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_float
            _C_LIB.void_oracle_spmm_int8.restype = ctypes.c_int
            _C_LIB.void_oracle_spmm_int8.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, f32, vp, vp, vp]
    return _C_LIB or None


def spmm_int8_c(values_q, scales, block_rows, block_cols, shape, b_q, b_scale=1.0, col_scale=None, want_acc=False):
    """spmm_int8 (and, with want_acc, spmm_int8_acc) through the C restatement: int8 x int8 -> int32 arithmetic,
    OpenMP over tile rows.  Same results as the numpy functions above; raises RuntimeError without the library."""
    lib = c_library()
    if lib is None:
        raise RuntimeError("the C oracle is not available (no C compiler and no prebuilt library)")
    nbr, nbc, row_ptr, bidx = _row_order(block_rows, block_cols, shape)
    M, K = shape
    N = b_q.shape[1]
    vals = np.ascontiguousarray(values_q, dtype=np.int8)
    sc = np.ascontiguousarray(scales, dtype=np.float32)
    bc = np.ascontiguousarray(block_cols, dtype=np.int32)
    b = np.ascontiguousarray(b_q, dtype=np.int8)
    cs = None if col_scale is None else np.ascontiguousarray(col_scale, dtype=np.float32)
    out = np.empty((M, N), dtype=np.float32)
    acc = np.empty((nbr * TILE, N), dtype=np.int32) if want_acc else None
    ptr = lambda a: None if a is None else a.ctypes.data
    lib.void_oracle_spmm_int8(ptr(vals), ptr(sc), ptr(bc), ptr(row_ptr), ptr(bidx), nbr, M, K, N, ptr(b),
                              float(b_scale), ptr(cs), ptr(acc), ptr(out))
    return (out, acc) if want_acc else out


def spmm_fp8(values_fp8, scales, block_rows, block_cols, shape, b, per_tensor=False):
    """fp32 result of void_spmm_fp8_kernel, void/fp8.py:624-659: for every tile of the row, in row
    order, acc += (float(A8) * scale) @ float(B block), all in fp32.  ``b`` is fp32 [K, N]."""
    nbr, nbc, row_ptr, bidx = _row_order(block_rows, block_cols, shape)
    M, K = shape
    N = b.shape[1]
    a = fp8_bytes_to_float(values_fp8).astype(np.float32)
    bf = np.asarray(b, dtype=np.float32)
    out = np.zeros((nbr * TILE, N), dtype=np.float32)
    for r in range(nbr):
        acc = np.zeros((TILE, N), dtype=np.float32)
        for i in bidx[int(row_ptr[r]):int(row_ptr[r + 1])]:
            s = np.float32(scales[0] if per_tensor else scales[i])
            acc = acc + np.matmul(a[i] * s, _b_block(bf, int(block_cols[i]), K))
        out[r * TILE:(r + 1) * TILE] = acc
    return out[:M]


def gelu_tanh_sigmoid(x):
    """_gelu of void/fusion.py:38-43 in fp32: x * 0.5 * (1 + (2*sigmoid(2u) - 1)),
    u = 0.7978845608 * (x + 0.044715 x^3)."""
    x = np.asarray(x, dtype=np.float32)
    inner = np.float32(0.7978845608) * (x + np.float32(0.044715) * x * x * x)
    sig = np.float32(1.0) / (np.float32(1.0) + np.exp(-(np.float32(2.0) * inner)))
    t = np.float32(2.0) * sig - np.float32(1.0)
    return (x * np.float32(0.5) * (np.float32(1.0) + t)).astype(np.float32)


def spmm_backward(values, block_rows, block_cols, shape, b, grad_c):
    """VOIDSpMMFunction.backward, void/autograd.py:160-221, in fp32: dL/dB = A^T @ dL/dC as the SpMM of the
    transposed tensor (tiles transposed, block rows and columns swapped, :178-191); dL/dA_values[i] =
    dL/dC[32 br : 32 br + 32, :] @ B[32 bc : 32 bc + 32, :]^T for the stored tiles only (:14-96), rows of dL/dC
    and of B beyond the matrix read as zero (boundary_check)."""
    M, K = shape
    a = np.asarray(values, dtype=np.float32)
    g = np.asarray(grad_c, dtype=np.float32)
    bf = np.asarray(b, dtype=np.float32)
    grad_b = spmm_fp(np.ascontiguousarray(a.transpose(0, 2, 1)), block_cols, block_rows, (K, M), g)
    grad_values = np.zeros_like(a)
    for i in range(len(block_rows)):
        grad_values[i] = np.matmul(_b_block(g, int(block_rows[i]), M), _b_block(bf, int(block_cols[i]), K).T)
    return grad_values, grad_b


def silu(x):
    """_silu of void/fusion.py:53-56: x * sigmoid(x) in fp32."""
    x = np.asarray(x, dtype=np.float32)
    return (x * (np.float32(1.0) / (np.float32(1.0) + np.exp(-x)))).astype(np.float32)


def sparse_mlp(w1, w2, x, bias1=None, bias2=None, act=gelu_tanh_sigmoid):
    """fused_sparse_mlp, void/fusion.py:557-602: y = (W2 @ act(W1 @ x^T + b1[:, None]) + b2[:, None])^T with the
    row-bias kernel of :201-304 for both layers.  w1 / w2 = (values, block_rows, block_cols, shape); x [batch, in]."""
    h = spmm_fp(*w1, np.ascontiguousarray(np.asarray(x, dtype=np.float32).T))
    if bias1 is not None:
        h = h + np.asarray(bias1, dtype=np.float32)[:, None]
    h = act(h)
    y = spmm_fp(*w2, h)
    if bias2 is not None:
        y = y + np.asarray(bias2, dtype=np.float32)[:, None]
    return np.ascontiguousarray(y.T)


# ----------------------------------------------------------------------------- Stream-K
def stream_k_workload(row_ptr, n_blocks, n_workers=None, max_work_per_worker=16):
    """The worker table of compute_stream_k_workload, void/stream_k.py:55-110.
    Returns (worker_rows, block_start, block_end, needs_atomic) as int32/int32/int32/bool."""
    total = int(n_blocks)
    if n_workers is None:
        n_workers = min(total, 1024)
    target = (total + n_workers - 1) // n_workers      # ZeroDivisionError when total == 0, like :66
    target = min(target, max_work_per_worker)
    rows, starts, ends, atomic = [], [], [], []
    for r in range(len(row_ptr) - 1):
        rs, re = int(row_ptr[r]), int(row_ptr[r + 1])
        pos = rs
        while pos < re:
            n = min(target, re - pos)
            rows.append(r)
            starts.append(pos)
            ends.append(pos + n)
            atomic.append(pos > rs or pos + n < re)
            pos += n
    return (np.asarray(rows, dtype=np.int32), np.asarray(starts, dtype=np.int32),
            np.asarray(ends, dtype=np.int32), np.asarray(atomic, dtype=bool))


def workload_balance(row_ptr):
    """analyze_workload_balance, void/stream_k.py:467-492 (torch .std() is the unbiased one)."""
    work = np.diff(np.asarray(row_ptr)).astype(np.float32)
    nz = work[work > 0]
    if len(nz) == 0:
        return {"empty": True}
    t = torch.from_numpy(nz)
    return {
        "empty": False,
        "n_rows": len(work),
        "n_nonempty_rows": int((work > 0).sum()),
        "min_blocks_per_row": float(t.min()),
        "max_blocks_per_row": float(t.max()),
        "mean_blocks_per_row": float(t.mean()),
        "std_blocks_per_row": float(t.std()),
        "imbalance_ratio": float(t.max() / t.mean()),
        "coefficient_of_variation": float(t.std() / t.mean()),
    }


# ----------------------------------------------------------------------------- sharding
def shard_rows(block_rows, nbr, world_size, rank):
    """ROW_WISE shard of shard_void_tensor, void/distributed.py:115-125, :150-161, :170-172:
    rows_per_rank = ceil(nbr / world); rank owns block rows [start, end); kept tiles stay in their
    original (Morton) order and get block_rows - start.  A rank past the end gets start > end and no
    tiles, as in the reference.  Pinned by shard_small.npz (reference output)."""
    rpr = (nbr + world_size - 1) // world_size
    start = rank * rpr
    end = min(start + rpr, nbr)
    block_rows = np.asarray(block_rows)
    mask = (block_rows >= start) & (block_rows < end)
    idx = np.nonzero(mask)[0]
    return start, end, idx, (block_rows[idx] - start).astype(np.int32)


def shard(block_rows, block_cols, shape, world_size, rank, strategy, tile=32):
    """shard_void_tensor for the three strategies, void/distributed.py:112-172.
    ROW_WISE (:115-125): block rows [rank * ceil(nbr / world), ...), rows rebased (:160-161).
    COLUMN_WISE (:127-137): block columns [rank * ceil(nbc / world), ...); block_cols are NOT rebased
    (only rows are, :159-161) although the local shape shrinks to the range (:174-176).
    BLOCK_WISE (:139-145): tile i of the stored order goes to rank i % world; ranges span the grid.
    Returns a dict: ids (kept positions, stored order), rows, cols, row_range, col_range, shape."""
    block_rows, block_cols = np.asarray(block_rows), np.asarray(block_cols)
    M, K = int(shape[0]), int(shape[1])
    nbr, nbc = (M + tile - 1) // tile, (K + tile - 1) // tile
    if strategy == "row_wise":
        start, end, idx, rows = shard_rows(block_rows, nbr, world_size, rank)
        return {"ids": idx, "rows": rows, "cols": block_cols[idx].astype(np.int32), "row_range": (start, end),
                "col_range": (0, nbc), "shape": ((end - start) * tile, K)}
    if strategy == "column_wise":
        cpr = (nbc + world_size - 1) // world_size
        start = rank * cpr
        end = min(start + cpr, nbc)
        idx = np.nonzero((block_cols >= start) & (block_cols < end))[0]
        return {"ids": idx, "rows": block_rows[idx].astype(np.int32), "cols": block_cols[idx].astype(np.int32),
                "row_range": (0, nbr), "col_range": (start, end), "shape": (M, (end - start) * tile)}
    if strategy == "block_wise":
        idx = np.nonzero(np.arange(len(block_rows)) % world_size == rank)[0]
        return {"ids": idx, "rows": block_rows[idx].astype(np.int32), "cols": block_cols[idx].astype(np.int32),
                "row_range": (0, nbr), "col_range": (0, nbc), "shape": (M, K)}
    raise ValueError("Unknown sharding strategy: %s" % strategy)
