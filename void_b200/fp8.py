"""FP8 (E4M3) quantisation and FP8 SpMM for VOID tensors on B200.

Mirrors the public surface of void/fp8.py: FP8Format / FP8Config (:15-66), FP8ScalingInfo
(:69-105), create_scaling_info (:108-152), compute_amax (:159-182), quantize_to_fp8 (:185-229),
dequantize_from_fp8 (:232-257), FP8VOIDTensor (:438-570), void_spmm_fp8 (:674-742) and
void_tensor_to_fp8 (:749-766).

What differs from the reference, and why: its kernel converts the FP8 tile to fp32, multiplies it
by the block's scale and runs an fp32 dot against a floating-point B (:638-659).  On B200 the
FP8 product runs on the FP8 tensor cores (tcgen05 kind::f8f6f4), which need BOTH operands in FP8, so it
takes B as E4M3 with one scale per column (quantize_cols_fp8); the column scales are applied once in
the epilogue (they factor out of the sum), A's per-tile scales either folded into A when it is packed
or applied to every tile's fp32 product (scale_terms of void_spmm_fp8).  A floating-point B handed to
void_spmm_fp8 stays in floating point as in the reference: the tiles are dequantised once and the
floating-point kernel runs.
"""
from dataclasses import dataclass, field
from enum import Enum
from typing import Literal, Optional, Tuple, Union

import torch

from . import _lib, _spmm


class FP8Format(Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"


FP8_MAX = {FP8Format.E4M3: 448.0, FP8Format.E5M2: 57344.0}
FP8_MIN = {FP8Format.E4M3: -448.0, FP8Format.E5M2: -57344.0}


@dataclass
class FP8Config:
    """FP8 settings (void/fp8.py:37-66).  The B200 kernels implement E4M3."""
    format: FP8Format = FP8Format.E4M3
    scale_mode: Literal["per_tensor", "per_block", "per_row"] = "per_tensor"
    margin: float = 0.0
    amax_history_len: int = 16

    @property
    def max_value(self) -> float:
        return FP8_MAX[self.format]

    @property
    def torch_dtype(self) -> torch.dtype:
        return torch.float8_e4m3fn if self.format == FP8Format.E4M3 else torch.float8_e5m2


@dataclass
class FP8ScalingInfo:
    """Scale factors and amax history of an FP8 tensor (void/fp8.py:69-105)."""
    scale: torch.Tensor
    scale_inv: torch.Tensor
    amax: torch.Tensor
    amax_history: torch.Tensor
    config: FP8Config = field(default_factory=FP8Config)

    def update_amax(self, new_amax: torch.Tensor) -> None:
        self.amax_history = torch.roll(self.amax_history, shifts=1, dims=-1)
        if self.amax_history.dim() == 1:
            self.amax_history[0] = new_amax
        else:
            self.amax_history[..., 0] = new_amax
        self.amax = new_amax

    def compute_scale(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.amax_history.dim() == 1:
            smoothed = self.amax_history.max()
        else:
            smoothed = self.amax_history.max(dim=-1).values
        fp8_max = self.config.max_value * (1.0 - self.config.margin)
        self.scale = torch.clamp(smoothed / fp8_max, min=1e-12)
        self.scale_inv = 1.0 / self.scale
        return self.scale, self.scale_inv


def create_scaling_info(shape, config: FP8Config, device="cuda") -> FP8ScalingInfo:
    """Unit-scale FP8ScalingInfo for a tensor shape (void/fp8.py:108-152)."""
    if config.scale_mode == "per_tensor":
        scale_shape = ()
    elif config.scale_mode in ("per_block", "per_row"):
        scale_shape = (shape[0],)
    else:
        raise ValueError(f"Unknown scale_mode: {config.scale_mode}")
    hist_shape = (config.amax_history_len,) if scale_shape == () else scale_shape + (config.amax_history_len,)
    return FP8ScalingInfo(scale=torch.ones(scale_shape, dtype=torch.float32, device=device),
                          scale_inv=torch.ones(scale_shape, dtype=torch.float32, device=device),
                          amax=torch.zeros(scale_shape, dtype=torch.float32, device=device),
                          amax_history=torch.zeros(hist_shape, dtype=torch.float32, device=device), config=config)


def compute_amax(tensor: torch.Tensor, scale_mode: str = "per_tensor") -> torch.Tensor:
    """Absolute maxima for scaling (void/fp8.py:159-182)."""
    if scale_mode == "per_tensor":
        return tensor.abs().max()
    if scale_mode in ("per_block", "per_row"):
        return tensor.reshape(tensor.shape[0], -1).abs().max(dim=1).values
    raise ValueError(f"Unknown scale_mode: {scale_mode}")


def _fresh_info(config, scale, scale_inv, amax) -> FP8ScalingInfo:
    """Scaling info after the first quantize_to_fp8 call: history = [amax, 0, 0, ...]."""
    hist = torch.zeros(tuple(amax.shape) + (config.amax_history_len,), dtype=torch.float32, device=amax.device)
    hist[..., 0] = amax
    return FP8ScalingInfo(scale=scale, scale_inv=scale_inv, amax=amax, amax_history=hist, config=config)


def quantize_cols_fp8(b: torch.Tensor):
    """Per-column E4M3 of a [K, N] matrix -> (float8_e4m3fn [K, N], scale [N], scale_inv [N]).
    Same numbers as quantize_to_fp8(b.T, scale_mode='per_row') transposed back."""
    _lib.require_cuda(b)
    lib = _lib.load()
    K, N = b.shape
    bf = b.to(torch.float32).contiguous()
    ld = (N + 15) // 16 * 16
    q = torch.empty(K, ld, dtype=torch.uint8, device=b.device)
    scale = torch.empty(N, dtype=torch.float32, device=b.device)
    scale_inv = torch.empty(N, dtype=torch.float32, device=b.device)
    with torch.cuda.device(b.device):
        _lib.check(lib.void_quant_cols(_lib.ptr(bf), bf.stride(0), K, N, _lib.KIND_F8E4M3, _lib.ptr(q), ld,
                                       _lib.ptr(scale), _lib.ptr(scale_inv), _lib.stream_ptr(b.device)),
                   "void_quant_cols")
    return q.view(torch.float8_e4m3fn)[:, :N], scale, scale_inv


def quantize_to_fp8(tensor: torch.Tensor, config: Optional[FP8Config] = None,
                    scaling_info: Optional[FP8ScalingInfo] = None):
    """Quantise to FP8 (void/fp8.py:185-229).  Implemented for the two shapes the SpMM path uses:
    per_block over [n_blocks, 32, 32] tiles and per_row over a 2-D matrix, with a fresh history
    (scale = amax / 448)."""
    if config is None:
        config = FP8Config()
    if config.format != FP8Format.E4M3:
        raise NotImplementedError("void_b200 implements E4M3 only (the format its tensor-core path uses)")
    if scaling_info is not None:
        raise NotImplementedError("delayed scaling from an existing amax history is outside the SpMM path")
    _lib.require_cuda(tensor)
    lib = _lib.load()
    dev = tensor.device
    if config.scale_mode == "per_block" and tensor.dim() == 3 and tuple(tensor.shape[1:]) == (32, 32):
        n = tensor.shape[0]
        vf = tensor.to(torch.float32).contiguous()
        q = torch.empty(n, 32, 32, dtype=torch.uint8, device=dev)
        scale = torch.empty(n, dtype=torch.float32, device=dev)
        scale_inv = torch.empty(n, dtype=torch.float32, device=dev)
        amax = torch.empty(n, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.void_quant_fp8_tiles(_lib.ptr(vf), n, _lib.ptr(q), _lib.ptr(scale), _lib.ptr(scale_inv),
                                                _lib.ptr(amax), _lib.stream_ptr(dev)), "void_quant_fp8_tiles")
        return q.view(torch.float8_e4m3fn), _fresh_info(config, scale, scale_inv, amax)
    if config.scale_mode == "per_block" and tensor.dim() >= 2:
        # one scale per slice of the first dimension (void/fp8.py:97-99): the per-row case of the flattened slices
        flat = tensor.reshape(tensor.shape[0], -1)
        q_t, scale, scale_inv = quantize_cols_fp8(flat.t())
        amax = compute_amax(tensor, "per_block")
        return q_t.t().contiguous().reshape(tensor.shape), _fresh_info(config, scale, scale_inv, amax)
    if config.scale_mode == "per_row" and tensor.dim() == 2:
        q_t, scale, scale_inv = quantize_cols_fp8(tensor.t())
        amax = compute_amax(tensor, "per_row")
        return q_t.t().contiguous(), _fresh_info(config, scale, scale_inv, amax)
    if config.scale_mode == "per_tensor":
        # one scale for everything: quantise the flattened tensor as a single column
        flat = tensor.reshape(-1, 1)
        q, scale, scale_inv = quantize_cols_fp8(flat)
        amax = compute_amax(tensor, "per_tensor")
        return q.contiguous().reshape(tensor.shape), _fresh_info(config, scale.reshape(()), scale_inv.reshape(()), amax)
    raise NotImplementedError("quantize_to_fp8: unsupported (scale_mode, shape) = (%s, %s)"
                              % (config.scale_mode, tuple(tensor.shape)))


def dequantize_from_fp8(tensor: torch.Tensor, scaling_info: FP8ScalingInfo,
                        output_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """x = float(q) * scale (void/fp8.py:232-257)."""
    f = tensor.to(torch.float32)
    if scaling_info.config.scale_mode == "per_tensor":
        res = f * scaling_info.scale
    else:
        res = f * scaling_info.scale.view((tensor.shape[0],) + (1,) * (tensor.dim() - 1))
    return res.to(output_dtype)


@dataclass
class FP8VOIDTensor:
    """VOID tensor with FP8 storage (void/fp8.py:438-570)."""
    values_fp8: torch.Tensor
    scaling_info: FP8ScalingInfo
    block_rows: torch.Tensor
    block_cols: torch.Tensor
    morton_codes: torch.Tensor
    shape: Tuple[int, int]
    tile_size: Tuple[int, int]
    nnz_original: int
    n_blocks: int
    density: float

    @classmethod
    def from_void_tensor(cls, void_tensor, config: Optional[FP8Config] = None) -> "FP8VOIDTensor":
        if config is None:
            config = FP8Config(scale_mode="per_block")
        values_fp8, info = quantize_to_fp8(void_tensor.values, config=config)
        return cls(values_fp8=values_fp8, scaling_info=info, block_rows=void_tensor.block_rows,
                   block_cols=void_tensor.block_cols, morton_codes=void_tensor.morton_codes, shape=void_tensor.shape,
                   tile_size=void_tensor.tile_size, nnz_original=void_tensor.nnz_original,
                   n_blocks=void_tensor.n_blocks, density=void_tensor.density)

    def to_void_tensor(self, output_dtype: torch.dtype = torch.float16):
        from .format import VOIDTensor
        values = dequantize_from_fp8(self.values_fp8, self.scaling_info, output_dtype=output_dtype)
        return VOIDTensor(values=values, block_rows=self.block_rows, block_cols=self.block_cols,
                          morton_codes=self.morton_codes, shape=self.shape, tile_size=self.tile_size,
                          nnz_original=self.nnz_original, n_blocks=self.n_blocks, density=self.density,
                          dtype=output_dtype)

    def to(self, device) -> "FP8VOIDTensor":
        s = self.scaling_info
        return FP8VOIDTensor(
            values_fp8=self.values_fp8.to(device),
            scaling_info=FP8ScalingInfo(s.scale.to(device), s.scale_inv.to(device), s.amax.to(device),
                                        s.amax_history.to(device), s.config),
            block_rows=self.block_rows.to(device), block_cols=self.block_cols.to(device),
            morton_codes=self.morton_codes.to(device), shape=self.shape, tile_size=self.tile_size,
            nnz_original=self.nnz_original, n_blocks=self.n_blocks, density=self.density)

    def cuda(self) -> "FP8VOIDTensor":
        return self.to("cuda")

    @property
    def block_grid(self) -> Tuple[int, int]:
        return ((self.shape[0] + self.tile_size[0] - 1) // self.tile_size[0],
                (self.shape[1] + self.tile_size[1] - 1) // self.tile_size[1])

    @property
    def memory_bytes(self) -> int:
        return (self.values_fp8.numel() + self.scaling_info.scale.numel() * 4 +
                (self.block_rows.numel() + self.block_cols.numel()) * 4)

    def packed(self) -> _spmm.PackedTiles:
        """The tile-row-major packed copy the kernels stream (built once, cached)."""
        return _spmm.cached_pack(self, self.values_fp8.view(torch.uint8), self.scaling_info.scale, self.block_rows,
                                 self.block_cols, self.shape, _lib.KIND_F8E4M3)

    def packed_split(self, terms: int) -> _spmm.PackedTiles:
        """Packed copy with the tile scales folded in: every tile as a sum of ``terms`` E4M3 tiles relative to
        the largest scale of its tile row (built once per ``terms``, cached)."""
        v, sc = self.values_fp8.view(torch.uint8), self.scaling_info.scale
        key = (terms, v.data_ptr(), v._version, sc.data_ptr(), sc._version, self.block_rows.data_ptr(),
               self.block_cols.data_ptr(), str(v.device), tuple(self.shape))
        cache = self.__dict__.setdefault("_packed_split_cache", {})
        p = cache.get(terms)
        if p is None or p.key != key:
            p = _spmm._mark_ready(_spmm.pack_f8_split(v, sc, self.block_rows, self.block_cols, self.shape, terms))
            p.key = key
            cache[terms] = p
        return p

    def __repr__(self) -> str:
        return (f"FP8VOIDTensor(shape={self.shape}, tile_size={self.tile_size}, n_blocks={self.n_blocks}, "
                f"format={self.scaling_info.config.format.value}, scale_mode={self.scaling_info.config.scale_mode})")


DEFAULT_SCALE_TERMS = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 3}


def void_spmm_fp8(a: FP8VOIDTensor, b: torch.Tensor, output_dtype: torch.dtype = torch.float16, *,
                  b_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  activation: int = 0, bias: Optional[torch.Tensor] = None,
                  scale_terms: Optional[int] = None) -> torch.Tensor:
    """FP8 sparse-dense product C = A @ B (void/fp8.py:674-742).

    a: FP8VOIDTensor [M, K];  b: [K, N], either float8_e4m3fn with ``b_scale`` = per-column scales [N]
    (quantize_cols_fp8; the FP8 tensor-core product), or floating point as in the reference (then A's tiles are
    dequantised and the floating-point kernel multiplies them with B as it is).  Returns [M, N] in
    ``output_dtype`` (default float16, as in the reference).

    ``scale_terms`` says how the per-tile scales of A (void/fp8.py:638-646) enter the sum:
      0     every tile's fp32 product is multiplied by its scale in registers before it is added (the per-tile
            kernel; exact in fp32, and the slow way: every product is read back from tensor memory);
      2, 3  the scales are folded into A when it is packed - a * scale / (largest scale of the tile row) stored
            as a sum of 2 or 3 E4M3 numbers - and the tensor cores accumulate whole tile rows (the row-accumulate
            kernel).  8 / 12 significant bits of that operand; measured against the exact form the results
            differ by 4e-4 / 2e-5 of max|C| (the bar of this path is 1e-2, one fp16 rounding is 3e-4).
      None  2 for 16-bit outputs, 3 for fp32 outputs.
    With one scale for all tiles (scale_mode="per_tensor") the folded factor is 1 and every form is exact.
    """
    assert b.dim() == 2
    assert a.shape[1] == b.shape[0]
    _lib.require_cuda(a.values_fp8, b)
    if a.scaling_info.config.format != FP8Format.E4M3:
        raise NotImplementedError("void_b200 implements E4M3 only")
    M, K = a.shape
    N = b.shape[1]
    if b.dtype != torch.float8_e4m3fn:
        # B in floating point stays in floating point, as in the reference kernel (void/fp8.py:648-659: the tile
        # is dequantised, B is loaded as it is, tl.dot multiplies them as TF32): the tiles are dequantised once
        # (cached on the tensor) and the floating-point kernel runs - TF32 for an fp32 B, exact 16-bit products
        # when B is fp16 / bf16.  The FP8 tensor-core product needs B in E4M3: pass quantize_cols_fp8(b) for that.
        from .ops import void_spmm
        if b_scale is not None:
            raise ValueError("b_scale belongs to an FP8 B")
        dt = b.dtype if b.dtype in (torch.float16, torch.bfloat16) else torch.float32
        cache = a.__dict__.setdefault("_dequantised", {})
        key = (a.values_fp8.data_ptr(), a.values_fp8._version, a.scaling_info.scale.data_ptr(), a.scaling_info.scale._version)
        hit = cache.get(dt)
        if hit is None or hit[0] != key:
            hit = cache[dt] = (key, a.to_void_tensor(dt))
        if out is None:
            out = torch.empty(M, N, dtype=output_dtype, device=b.device)
        return void_spmm(hit[1], b if b.dtype == dt else b.to(dt), out, activation=activation, bias=bias)
    b8, col_scale = b, (None if b_scale is None else b_scale.reshape(-1))
    if out is None:
        out = torch.empty(M, N, dtype=output_dtype, device=b.device)
    if scale_terms is None:
        scale_terms = DEFAULT_SCALE_TERMS[out.dtype]
    if scale_terms not in (0, 2, 3):
        raise ValueError("scale_terms must be 0, 2, 3 or None")
    if scale_terms == 0:
        return _spmm.spmm(a.packed(), b8.view(torch.uint8), out, scale_mode=_lib.SCALE_PER_TILE, col_scale=col_scale,
                          bias=bias, act=activation)
    return _spmm.spmm(a.packed_split(scale_terms), b8.view(torch.uint8), out, scale_mode=_lib.SCALE_ROW_MEAN,
                      col_scale=col_scale, bias=bias, act=activation)


def void_tensor_to_fp8(void_tensor, format: str = "e4m3", scale_mode: str = "per_block") -> FP8VOIDTensor:
    """VOIDTensor -> FP8VOIDTensor (void/fp8.py:749-766)."""
    fmt = FP8Format.E4M3 if format == "e4m3" else FP8Format.E5M2
    return FP8VOIDTensor.from_void_tensor(void_tensor, FP8Config(format=fmt, scale_mode=scale_mode))


__all__ = [
    "FP8Format", "FP8Config", "FP8ScalingInfo", "FP8VOIDTensor", "create_scaling_info", "compute_amax",
    "quantize_to_fp8", "dequantize_from_fp8", "void_spmm_fp8", "void_tensor_to_fp8", "quantize_cols_fp8",
]
