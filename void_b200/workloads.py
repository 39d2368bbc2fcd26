"""Seeded synthetic workloads with the shapes of the reference's block-sparse benchmark sweep
(benchmarks/bsr_comparison.py:42-55, :185-214: 4096x4096, 32x32 tiles, N = 512, uniformly random
block mask) and of the larger Stream-K and multi-GPU cases.  They stand in for the reference's
own benchmark inputs; tile values are N(0,1) (the per-block quantisation is scale invariant).

Everything is built without ever materialising a dense A: a boolean block mask, the tile values
of the active blocks, and a VOIDTensor assembled from them (void_from_block_mask).
"""
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .format import VOIDTensor, morton_encode_batch, void_from_block_mask
from .int_quant import Int8VOIDTensor, IntQuantConfig, quantize_void_tensor


@dataclass
class Workload:
    name: str
    a: VOIDTensor            # fp32 tiles (None when only the quantised form was generated)
    b: torch.Tensor          # fp32 [K, N]
    shape: tuple
    N: int
    nnz: int


def uniform_mask(nbr: int, nbc: int, block_sparsity: float, seed: int = 0) -> np.ndarray:
    """Uniformly random block mask: a block is kept when rng.random() > sparsity."""
    rng = np.random.default_rng(seed)
    return rng.random((nbr, nbc)) > block_sparsity


def zipf_mask(nbr: int, nbc: int, alpha: float = 1.5, cap: int = 512, mean_tiles: float = 15.36,
              seed: int = 0) -> np.ndarray:
    """Power-law tile-row lengths: counts ~ Zipf(alpha) capped at ``cap`` and rescaled to the wanted
    mean (15.36 of 512 columns = 97 % block sparsity), column positions uniform without replacement."""
    rng = np.random.default_rng(seed)
    z = np.minimum(rng.zipf(alpha, nbr), cap).astype(np.float64)
    counts = np.clip(np.rint(z * mean_tiles / z.mean()), 1, min(cap, nbc)).astype(np.int64)
    mask = np.zeros((nbr, nbc), dtype=bool)
    for r, c in enumerate(counts):
        mask[r, rng.choice(nbc, int(c), replace=False)] = True
    return mask


def block_sparse(mask: np.ndarray, N: int, seed: int = 0, device="cuda", name="custom") -> Workload:
    """VOIDTensor with N(0,1) tiles on ``mask`` plus an N(0,1) B of N columns."""
    nbr, nbc = mask.shape
    nnz = int(mask.sum())
    g = torch.Generator(device="cpu").manual_seed(seed)
    tiles = torch.randn(nnz, 32, 32, generator=g, dtype=torch.float32)
    b = torch.randn(nbc * 32, N, generator=g, dtype=torch.float32)
    a = void_from_block_mask(mask, tiles, device=device)
    return Workload(name, a, b.to(device), (nbr * 32, nbc * 32), N, nnz)


def headline(block_sparsity: float = 0.9, M: int = 4096, N: int = 512, seed: int = 0, device="cuda") -> Workload:
    """4096 x 4096, 32x32 tiles, uniform random block mask, N = 512."""
    nb = M // 32
    return block_sparse(uniform_mask(nb, nb, block_sparsity, seed), N, seed, device,
                        "uniform%d_bs%02d_n%d" % (M, round(block_sparsity * 100), N))


def power_law(M: int = 16384, N: int = 256, seed: int = 0, device="cuda") -> Workload:
    """16384 x 16384 with Zipf(1.5) tile-row lengths (about 97 % block sparsity), N = 256."""
    nb = M // 32
    mean = 15.36 * nb / 512
    return block_sparse(zipf_mask(nb, nb, 1.5, min(512, nb), mean, seed), N, seed, device, "zipf%d_n%d" % (M, N))


def sharded_int8(M: int = 65536, N: int = 1024, block_sparsity: float = 0.95, seed: int = 0, world_size: int = 1,
                 rank: int = 0, device="cuda", chunk_tiles: int = 16384):
    """INT8 row shard of the multi-GPU workload, generated directly on the device in chunks of
    tiles (N(0,1) -> per-block INT8), never as one fp32 tensor.  Every rank draws the same global
    mask from ``seed`` and keeps its own tile rows (the ROW_WISE ranges of shard_void_tensor).
    Returns (Int8VOIDTensor shard, (start_row, end_row), global nnz)."""
    from .distributed import row_range
    nbr = nbc = M // 32
    mask = uniform_mask(nbr, nbc, block_sparsity, seed)
    start, end = row_range(nbr, world_size, rank)
    rows, cols = np.nonzero(mask[start:end])
    codes = morton_encode_batch(rows + start, cols)      # Morton order of the global coordinates
    order = np.argsort(codes)
    rows, cols = rows[order], cols[order]
    n = len(rows)
    dev = torch.device(device)
    q = torch.empty(n, 32, 32, dtype=torch.int8, device=dev)
    scales = torch.empty(n, dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(seed * 1000003 + rank)
    for lo in range(0, n, chunk_tiles):
        hi = min(lo + chunk_tiles, n)
        vals = torch.randn(hi - lo, 32, 32, generator=g, dtype=torch.float32, device=dev)
        part = VOIDTensor(values=vals, block_rows=torch.zeros(hi - lo, dtype=torch.int32, device=dev),
                          block_cols=torch.zeros(hi - lo, dtype=torch.int32, device=dev),
                          morton_codes=torch.zeros(hi - lo, dtype=torch.int64, device=dev),
                          shape=(32, 32), tile_size=(32, 32), nnz_original=0, n_blocks=hi - lo, density=1.0)
        qp = quantize_void_tensor(part)
        q[lo:hi] = qp.values
        scales[lo:hi] = qp.scales
    shard = Int8VOIDTensor(values=q, scales=scales, zero_points=torch.zeros(n, dtype=torch.int8, device=dev),
                           block_rows=torch.as_tensor(rows.astype(np.int32), device=dev),
                           block_cols=torch.as_tensor(cols.astype(np.int32), device=dev),
                           shape=((end - start) * 32, M), tile_size=(32, 32), n_blocks=n, config=IntQuantConfig())
    return shard, (start, end), int(mask.sum())


def algorithmic_bytes(nnz: int, nbr: int, K: int, N: int, M: int, out_bytes: int, elem_bytes: int = 1) -> int:
    """Bytes one SpMM has to move at least: every stored tile with its column index (and, for the
    8-bit kinds, its scale), row_ptr, all of B (with its column scales for the 8-bit kinds), and C once."""
    scales = 4 if elem_bytes == 1 else 0
    return nnz * (1024 * elem_bytes + 4 + scales) + (nbr + 1) * 4 + K * N * elem_bytes + N * scales + M * N * out_bytes


def spmm_ops(nnz: int, N: int) -> int:
    """Multiply-adds x 2 over the stored tiles."""
    return 2 * nnz * 32 * 32 * N
