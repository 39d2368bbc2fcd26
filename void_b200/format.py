"""VOIDTensor format: block-sparse matrices stored as Morton-ordered dense 32x32 tiles.

Mirrors the public surface of void/format.py (VOIDTensor :54-80, morton_encode :15-25,
morton_encode_batch :41-51, csr_to_void :248-349, dense_to_void :352-446, get_row_block_info
:201-237) so that code written against the reference imports unchanged.  The tile index and, for
device="cuda", the format itself (kept tiles, Morton order, tile values) are built by the CUDA
library; there is no CPU compute path.
"""
import warnings
from dataclasses import dataclass
from typing import Tuple, Union

import numpy as np
import torch
from scipy import sparse

from . import _lib

MIN_TENSOR_CORE_TILE = 16


def morton_encode(x: int, y: int) -> int:
    """Morton (Z-order) code of a 2-D coordinate, x on the even bits (void/format.py:15-25)."""
    def spread_bits(v: int) -> int:
        v = (v | (v << 8)) & 0x00FF00FF
        v = (v | (v << 4)) & 0x0F0F0F0F
        v = (v | (v << 2)) & 0x33333333
        v = (v | (v << 1)) & 0x55555555
        return v
    return spread_bits(x) | (spread_bits(y) << 1)


def morton_decode(code: int) -> Tuple[int, int]:
    """Inverse of morton_encode (void/format.py:28-38)."""
    def compact_bits(v: int) -> int:
        v = v & 0x55555555
        v = (v | (v >> 1)) & 0x33333333
        v = (v | (v >> 2)) & 0x0F0F0F0F
        v = (v | (v >> 4)) & 0x00FF00FF
        v = (v | (v >> 8)) & 0x0000FFFF
        return v
    return compact_bits(code), compact_bits(code >> 1)


def morton_encode_batch(rows: np.ndarray, cols: np.ndarray) -> np.ndarray:
    """Vectorised Morton encoding (void/format.py:41-51)."""
    def spread_bits_vec(v: np.ndarray) -> np.ndarray:
        v = np.asarray(v).astype(np.uint64)
        for shift, mask in ((8, 0x00FF00FF), (4, 0x0F0F0F0F), (2, 0x33333333), (1, 0x55555555)):
            v = (v | (v << np.uint64(shift))) & np.uint64(mask)
        return v
    return spread_bits_vec(rows) | (spread_bits_vec(cols) << np.uint64(1))


def build_tile_index(block_rows: torch.Tensor, block_cols: torch.Tensor, nbr: int, nbc: int):
    """row_ptr[nbr+1] and block_indices[nnz] of a tile list on the GPU (void_build_tile_index)."""
    _lib.require_cuda(block_rows, block_cols)
    lib = _lib.load()
    dev = block_rows.device
    nnz = block_rows.numel()
    with torch.cuda.device(dev):
        row_ptr = torch.empty(nbr + 1, dtype=torch.int32, device=dev)
        block_indices = torch.empty(nnz, dtype=torch.int32, device=dev)
        ws_bytes = lib.void_tile_index_ws_bytes(nbr, nbc)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        br = block_rows.contiguous().to(torch.int32)
        bc = block_cols.contiguous().to(torch.int32)
        _lib.check(lib.void_build_tile_index(_lib.ptr(br), _lib.ptr(bc), nnz, nbr, nbc, _lib.ptr(row_ptr),
                                             _lib.ptr(block_indices), _lib.ptr(ws), ws_bytes, _lib.stream_ptr(dev)),
                   "void_build_tile_index")
        check_tile_index(row_ptr, nnz)
    return row_ptr, block_indices


def check_tile_index(row_ptr: torch.Tensor, nnz: int) -> None:
    """The index builder skips block coordinates outside the grid and counts a repeated (row, column) pair
    once; either shows as fewer indexed tiles than listed ones.  (One read of one integer per built index;
    the index is cached on its tensor.)"""
    indexed = int(row_ptr[-1].item())
    if indexed != nnz:
        raise ValueError("invalid VOID tile list: %d of %d tiles have block coordinates outside the block grid or "
                         "repeat an earlier (block_row, block_col) pair" % (nnz - indexed, nnz))


@dataclass
class VOIDTensor:
    """VOID sparse matrix (field for field the dataclass of void/format.py:54-80)."""
    values: torch.Tensor          # [n_blocks, tile_m, tile_n]
    block_rows: torch.Tensor      # [n_blocks] int32
    block_cols: torch.Tensor      # [n_blocks] int32
    morton_codes: torch.Tensor    # [n_blocks] int64
    shape: Tuple[int, int]
    tile_size: Tuple[int, int]
    nnz_original: int
    n_blocks: int
    density: float
    dtype: torch.dtype = torch.float32

    @property
    def padded_shape(self) -> Tuple[int, int]:
        tm, tn = self.tile_size
        return (((self.shape[0] + tm - 1) // tm) * tm, ((self.shape[1] + tn - 1) // tn) * tn)

    @property
    def block_grid(self) -> Tuple[int, int]:
        tm, tn = self.tile_size
        return ((self.shape[0] + tm - 1) // tm, (self.shape[1] + tn - 1) // tn)

    @property
    def sparsity(self) -> float:
        return 1.0 - (self.nnz_original / (self.shape[0] * self.shape[1]))

    @property
    def block_sparsity(self) -> float:
        return 1.0 - (self.n_blocks / (self.block_grid[0] * self.block_grid[1]))

    @property
    def overhead_ratio(self) -> float:
        return self.n_blocks * self.tile_size[0] * self.tile_size[1] / max(self.nnz_original, 1)

    def _replace_values(self, values, dtype=None, device=None):
        mv = (lambda t: t.to(device)) if device is not None else (lambda t: t)
        return VOIDTensor(values=values, block_rows=mv(self.block_rows), block_cols=mv(self.block_cols),
                          morton_codes=mv(self.morton_codes), shape=self.shape, tile_size=self.tile_size,
                          nnz_original=self.nnz_original, n_blocks=self.n_blocks, density=self.density,
                          dtype=self.dtype if dtype is None else dtype)

    def to(self, device: Union[str, torch.device]) -> "VOIDTensor":
        return self._replace_values(self.values.to(device), device=device)

    def cuda(self) -> "VOIDTensor":
        return self.to("cuda")

    def cpu(self) -> "VOIDTensor":
        return self.to("cpu")

    def to_dtype(self, dtype: torch.dtype) -> "VOIDTensor":
        return self._replace_values(self.values.to(dtype), dtype=dtype)

    def half(self) -> "VOIDTensor":
        return self.to_dtype(torch.float16)

    def bfloat16(self) -> "VOIDTensor":
        return self.to_dtype(torch.bfloat16)

    def float(self) -> "VOIDTensor":
        return self.to_dtype(torch.float32)

    def to_fp8(self, format: str = "e4m3", scale_mode: str = "per_block"):
        """FP8 copy of this tensor (void/format.py:169-184)."""
        from .fp8 import void_tensor_to_fp8
        return void_tensor_to_fp8(self, format=format, scale_mode=scale_mode)

    def to_dense(self) -> torch.Tensor:
        """Dense copy for validation (void/format.py:186-199), as one scatter instead of a loop."""
        tm, tn = self.tile_size
        nbr, nbc = self.block_grid
        out = torch.zeros(nbr, nbc, tm, tn, dtype=self.values.dtype, device=self.values.device)
        if self.n_blocks:
            out[self.block_rows.long(), self.block_cols.long()] = self.values
        out = out.permute(0, 2, 1, 3).reshape(nbr * tm, nbc * tn)
        return out[:self.shape[0], :self.shape[1]]

    def get_row_block_info(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(row_ptr, block_indices) as in void/format.py:201-237; cached on the object."""
        cached = getattr(self, "_row_ptr_cache", None)
        if cached is not None and cached.device == self.block_rows.device:
            return self._row_ptr_cache, self._block_indices_cache
        nbr, nbc = self.block_grid
        row_ptr, block_indices = build_tile_index(self.block_rows, self.block_cols, nbr, nbc)
        self._row_ptr_cache, self._block_indices_cache = row_ptr, block_indices
        return row_ptr, block_indices

    def __repr__(self) -> str:
        return (f"VOIDTensor(shape={self.shape}, tile_size={self.tile_size}, n_blocks={self.n_blocks}, "
                f"sparsity={self.sparsity:.1%}, block_sparsity={self.block_sparsity:.1%}, "
                f"overhead={self.overhead_ratio:.2f}x, dtype={self.dtype})")


def _build_on_device(mark, fill, M: int, N: int, dev, value_dtype: torch.dtype):
    """Shared tail of the device builders: mark kept tiles, read their count, emit the Morton-ordered
    index and fill the tile values.  Returns (values, block_rows, block_cols, morton_codes, n_blocks, nnz)."""
    lib = _lib.load()
    nbr, nbc = (M + 31) // 32, (N + 31) // 32
    with torch.cuda.device(dev):
        ws_bytes = lib.void_format_ws_bytes(nbr, nbc)
        if ws_bytes == 0:
            raise _lib.VoidB200Error("block grid %d x %d is too large for the device format builder" % (nbr, nbc))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        counts = torch.zeros(2, dtype=torch.int64, device=dev)
        mark(lib, ws, ws_bytes, counts)
        n_blocks, nnz = (int(v) for v in counts.tolist())          # the one synchronisation, like .nonzero()
        values = torch.empty(n_blocks, 32, 32, dtype=value_dtype, device=dev)
        block_rows = torch.empty(n_blocks, dtype=torch.int32, device=dev)
        block_cols = torch.empty(n_blocks, dtype=torch.int32, device=dev)
        codes = torch.empty(n_blocks, dtype=torch.int64, device=dev)
        _lib.check(lib.void_morton_emit(_lib.ptr(ws), nbr, nbc, n_blocks, _lib.ptr(block_rows), _lib.ptr(block_cols),
                                        _lib.ptr(codes), _lib.stream_ptr(dev)), "void_morton_emit")
        fill(lib, ws, n_blocks, block_rows, block_cols, values)
    return values, block_rows, block_cols, codes, n_blocks, nnz, nbr * nbc


def dense_to_void(matrix: torch.Tensor, tile_size: int = 32, threshold: float = 0.0) -> VOIDTensor:
    """Dense -> VOID on the GPU (void/format.py:352-446): tiles whose L1 norm exceeds ``threshold`` are kept,
    in ascending Morton order.  ``matrix`` is a CUDA tensor of float32, float16 or bfloat16."""
    assert matrix.dim() == 2, "Input must be 2D tensor"
    _lib.require_cuda(matrix)
    if tile_size != 32:
        raise NotImplementedError("void_b200 builds 32x32 tiles, got tile_size=%d" % tile_size)
    if matrix.dtype not in _lib.ELEM_CODE:
        raise _lib.VoidB200Error("dense_to_void takes float32, float16 or bfloat16, got %s" % matrix.dtype)
    M, N = matrix.shape
    dev = matrix.device
    a = matrix if matrix.stride(1) == 1 and matrix.stride(0) >= max(N, 1) else matrix.contiguous()
    elem, ld = _lib.ELEM_CODE[a.dtype], a.stride(0) if M > 1 else max(N, 1)

    def mark(lib, ws, ws_bytes, counts):
        _lib.check(lib.void_dense_mark(_lib.ptr(a), elem, ld, M, N, float(threshold), _lib.ptr(ws), ws_bytes,
                                       _lib.ptr(counts), _lib.stream_ptr(dev)), "void_dense_mark")

    def fill(lib, ws, n_blocks, block_rows, block_cols, values):
        _lib.check(lib.void_dense_gather(_lib.ptr(a), elem, ld, M, N, _lib.ptr(block_rows), _lib.ptr(block_cols),
                                         n_blocks, _lib.ptr(values), _lib.stream_ptr(dev)), "void_dense_gather")

    values, block_rows, block_cols, codes, n_blocks, nnz, grid = _build_on_device(mark, fill, M, N, dev, a.dtype)
    return VOIDTensor(values=values, block_rows=block_rows, block_cols=block_cols, morton_codes=codes, shape=(M, N),
                      tile_size=(32, 32), nnz_original=nnz, n_blocks=n_blocks,
                      density=(n_blocks / grid) if n_blocks else 0.0, dtype=a.dtype)


def _csr_to_void_device(matrix, dtype: torch.dtype, device) -> VOIDTensor:
    """csr_to_void with the CSR arrays uploaded and everything else done by the CUDA library."""
    M, N = matrix.shape
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    crow = torch.from_numpy(matrix.indptr.astype(np.int32)).to(dev)
    col = torch.from_numpy(matrix.indices.astype(np.int32)).to(dev)
    data = torch.from_numpy(matrix.data.astype(np.float32)).to(dev)

    def mark(lib, ws, ws_bytes, counts):
        _lib.check(lib.void_csr_mark(_lib.ptr(crow), _lib.ptr(col), M, N, _lib.ptr(ws), ws_bytes, _lib.ptr(counts),
                                     _lib.stream_ptr(dev)), "void_csr_mark")

    def fill(lib, ws, n_blocks, block_rows, block_cols, values):
        _lib.check(lib.void_csr_scatter(_lib.ptr(crow), _lib.ptr(col), _lib.ptr(data), M, N, _lib.ptr(ws), n_blocks,
                                        _lib.ptr(values), _lib.stream_ptr(dev)), "void_csr_scatter")

    values, block_rows, block_cols, codes, n_blocks, _, grid = _build_on_device(mark, fill, M, N, dev, torch.float32)
    if dtype != torch.float32:
        values = values.to(dtype)
    return VOIDTensor(values=values, block_rows=block_rows, block_cols=block_cols, morton_codes=codes, shape=(M, N),
                      tile_size=(32, 32), nnz_original=matrix.nnz, n_blocks=n_blocks, density=n_blocks / grid, dtype=dtype)


def csr_to_void(matrix, tile_size: int = 32, dtype: torch.dtype = torch.float32, device: str = "cpu",
                warn_small_tiles: bool = True) -> VOIDTensor:
    """CSR -> VOID (void/format.py:248-349): active blocks are those holding a stored entry,
    sorted by Morton code.  For a CUDA ``device`` and 32x32 tiles the CSR arrays are uploaded and the
    format is built there (void_csr_mark / void_morton_emit / void_csr_scatter); otherwise the
    per-nonzero Python loop of the reference (:321-327) is one vectorised numpy scatter, with the
    same "last write wins" result."""
    if warn_small_tiles and tile_size < MIN_TENSOR_CORE_TILE:
        warnings.warn(f"tile_size={tile_size} < {MIN_TENSOR_CORE_TILE}, Tensor Cores require K >= 16", UserWarning)
    if not sparse.isspmatrix_csr(matrix):
        matrix = sparse.csr_matrix(matrix)
    M, N = matrix.shape
    if tile_size == 32 and torch.device(device).type == "cuda" and M > 0 and N > 0 and matrix.has_canonical_format \
            and matrix.nnz < 2 ** 31:
        return _csr_to_void_device(matrix, dtype, device)
    nbr = (M + tile_size - 1) // tile_size
    nbc = (N + tile_size - 1) // tile_size
    coo = matrix.tocoo()
    rows, cols, data = coo.row.astype(np.int64), coo.col.astype(np.int64), coo.data
    block_keys = (rows // tile_size) * nbc + (cols // tile_size)
    unique_blocks, inverse = np.unique(block_keys, return_inverse=True)
    n_blocks = len(unique_blocks)
    active_rows, active_cols = unique_blocks // nbc, unique_blocks % nbc
    codes = morton_encode_batch(active_rows, active_cols)
    order = np.argsort(codes)
    new_index = np.zeros(n_blocks, dtype=np.int64)
    new_index[order] = np.arange(n_blocks)
    values = np.zeros((n_blocks, tile_size, tile_size), dtype=np.float32)
    values[new_index[inverse], rows % tile_size, cols % tile_size] = data
    values_t = torch.tensor(values, dtype=torch.float32, device=device)
    if dtype != torch.float32:
        values_t = values_t.to(dtype)
    return VOIDTensor(
        values=values_t,
        block_rows=torch.tensor(active_rows[order], dtype=torch.int32, device=device),
        block_cols=torch.tensor(active_cols[order], dtype=torch.int32, device=device),
        morton_codes=torch.tensor(codes[order].astype(np.int64), dtype=torch.int64, device=device),
        shape=(M, N), tile_size=(tile_size, tile_size), nnz_original=matrix.nnz, n_blocks=n_blocks,
        density=n_blocks / (nbr * nbc), dtype=dtype)


def void_from_block_mask(mask: np.ndarray, tile_values: torch.Tensor, shape=None, device="cuda") -> VOIDTensor:
    """Builds a VOIDTensor straight from a boolean block mask and its tile values (given in
    row-major order of the mask), Morton-sorted like csr_to_void.  The reference fills tiles with a
    Python loop per nonzero (void/format.py:321-327), which is unusable for the large benchmark
    inputs; this constructor yields the same fields without going through CSR."""
    nbr, nbc = mask.shape
    rows, cols = np.nonzero(mask)
    codes = morton_encode_batch(rows, cols)
    order = np.argsort(codes)
    n = len(rows)
    tm, tn = tile_values.shape[1], tile_values.shape[2]
    shape = shape or (nbr * tm, nbc * tn)
    values = tile_values[torch.as_tensor(order, device=tile_values.device)].to(device)
    nnz = int(torch.count_nonzero(values).item()) if n else 0
    return VOIDTensor(
        values=values,
        block_rows=torch.tensor(rows[order], dtype=torch.int32, device=device),
        block_cols=torch.tensor(cols[order], dtype=torch.int32, device=device),
        morton_codes=torch.tensor(codes[order].astype(np.int64), dtype=torch.int64, device=device),
        shape=shape, tile_size=(tm, tn), nnz_original=nnz, n_blocks=n, density=n / (nbr * nbc),
        dtype=values.dtype)
