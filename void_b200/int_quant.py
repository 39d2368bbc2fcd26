"""INT8 quantisation and INT8 SpMM for VOID tensors on B200.

Mirrors the public surface of void/int_quant.py: the enums and IntQuantConfig (:12-80),
QuantizationParams (:83-102), Int8VOIDTensor (:105-175), quantize_tensor (:254-305),
quantize_void_tensor (:328-388) and void_spmm_int8 (:543-612).  The arithmetic runs in the CUDA
library: per-tile / per-column / per-tensor quantisers and the tcgen05 SpMM kernel.

Semantics kept from the reference on purpose:
* symmetric scale = absmax / 128 (max(|qmin|, qmax), :204), q = round-half-even(x / scale)
  clamped to [-128, 127];
* void_spmm_int8 accumulates a whole tile row in int32 and multiplies by the MEAN of the row's
  a_scale * b_scale (:479-481, :516-526) - not by each block's own scale.  ``exact_scales=True``
  (an extension) applies every block's own scale instead.
Extensions that BASELINE workloads need (defaults reproduce the reference): ``b_scale`` may be a
per-column tensor [N]; ``out_dtype`` / ``out`` may be fp16 or bf16.
"""
from dataclasses import dataclass
from enum import Enum
from typing import Literal, Optional, Tuple, Union

import torch

from . import _lib, _spmm


class IntFormat(Enum):
    INT8 = "int8"
    UINT8 = "uint8"
    INT4 = "int4"
    UINT4 = "uint4"


class ScaleMode(Enum):
    PER_TENSOR = "per_tensor"
    PER_CHANNEL = "per_channel"
    PER_BLOCK = "per_block"


@dataclass
class IntQuantConfig:
    """Quantisation settings (void/int_quant.py:27-80).  The B200 kernels implement the default:
    INT8, symmetric, min-max calibration."""
    format: IntFormat = IntFormat.INT8
    symmetric: bool = True
    scale_mode: ScaleMode = ScaleMode.PER_BLOCK
    calibration_method: Literal["minmax", "percentile", "mse"] = "minmax"
    percentile: float = 99.9

    @property
    def bits(self) -> int:
        return 8 if self.format in (IntFormat.INT8, IntFormat.UINT8) else 4

    @property
    def is_signed(self) -> bool:
        return self.format in (IntFormat.INT8, IntFormat.INT4)

    @property
    def qmin(self) -> int:
        return {IntFormat.INT8: -128, IntFormat.UINT8: 0, IntFormat.INT4: -8, IntFormat.UINT4: 0}[self.format]

    @property
    def qmax(self) -> int:
        return {IntFormat.INT8: 127, IntFormat.UINT8: 255, IntFormat.INT4: 7, IntFormat.UINT4: 15}[self.format]


def _require_supported(config: IntQuantConfig):
    if config.format != IntFormat.INT8 or not config.symmetric or config.calibration_method != "minmax":
        raise NotImplementedError(
            "void_b200 implements symmetric min-max INT8 only (the configuration the SpMM kernel of the "
            "reference honours: it ignores zero points and never packs INT4)")


@dataclass
class QuantizationParams:
    scale: torch.Tensor
    zero_point: torch.Tensor
    config: IntQuantConfig
    original_shape: Tuple[int, ...]

    def to(self, device) -> "QuantizationParams":
        return QuantizationParams(self.scale.to(device), self.zero_point.to(device), self.config, self.original_shape)


@dataclass
class Int8VOIDTensor:
    """Quantised VOID tensor (void/int_quant.py:105-175)."""
    values: torch.Tensor        # int8 [n_blocks, tile_m, tile_k]
    scales: torch.Tensor        # float32 [n_blocks]
    zero_points: torch.Tensor   # int8 [n_blocks]
    block_rows: torch.Tensor
    block_cols: torch.Tensor
    shape: Tuple[int, int]
    tile_size: Tuple[int, int]
    n_blocks: int
    config: IntQuantConfig
    _row_ptr: Optional[torch.Tensor] = None
    _block_indices: Optional[torch.Tensor] = None

    @property
    def device(self) -> torch.device:
        return self.values.device

    @property
    def dtype(self) -> torch.dtype:
        return self.values.dtype

    @property
    def block_grid(self) -> Tuple[int, int]:
        return ((self.shape[0] + self.tile_size[0] - 1) // self.tile_size[0],
                (self.shape[1] + self.tile_size[1] - 1) // self.tile_size[1])

    def to(self, device) -> "Int8VOIDTensor":
        return Int8VOIDTensor(self.values.to(device), self.scales.to(device), self.zero_points.to(device),
                              self.block_rows.to(device), self.block_cols.to(device), self.shape, self.tile_size,
                              self.n_blocks, self.config)

    def cuda(self) -> "Int8VOIDTensor":
        return self.to("cuda")

    def get_row_block_info(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(row_ptr, block_indices), cached (void/int_quant.py:158-175)."""
        if self._row_ptr is None or self._block_indices is None or self._row_ptr.device != self.block_rows.device:
            from .format import build_tile_index
            nbr, nbc = self.block_grid
            self._row_ptr, self._block_indices = build_tile_index(self.block_rows, self.block_cols, nbr, nbc)
        return self._row_ptr, self._block_indices

    def packed(self) -> _spmm.PackedTiles:
        """The tile-row-major packed copy the kernels stream (built once, cached)."""
        p = _spmm.cached_pack(self, self.values, self.scales, self.block_rows, self.block_cols, self.shape,
                              _lib.KIND_I8)
        self._row_ptr, self._block_indices = p.row_ptr, p.block_indices
        return p


def quantize_cols_int8(b: torch.Tensor):
    """Per-column symmetric INT8 of a [K, N] matrix -> (int8 [K, N], float32 scales [N]).
    Same numbers as quantize_tensor(b.T, PER_CHANNEL) transposed back."""
    _lib.require_cuda(b)
    lib = _lib.load()
    K, N = b.shape
    bf = b.to(torch.float32).contiguous()
    ld = (N + 15) // 16 * 16
    q = torch.empty(K, ld, dtype=torch.int8, device=b.device)
    scale = torch.empty(N, dtype=torch.float32, device=b.device)
    with torch.cuda.device(b.device):
        _lib.check(lib.void_quant_cols(_lib.ptr(bf), bf.stride(0), K, N, _lib.KIND_I8, _lib.ptr(q), ld, _lib.ptr(scale),
                                       None, _lib.stream_ptr(b.device)), "void_quant_cols")
    return q[:, :N], scale


def _quantize_matrix_per_tensor(b: torch.Tensor):
    lib = _lib.load()
    K, N = b.shape
    bf = b.to(torch.float32).contiguous()
    ld = (N + 15) // 16 * 16
    q = torch.empty(K, ld, dtype=torch.int8, device=b.device)
    scale = torch.empty(1, dtype=torch.float32, device=b.device)
    with torch.cuda.device(b.device):
        _lib.check(lib.void_quant_i8_tensor(_lib.ptr(bf), bf.stride(0), K, N, _lib.ptr(q), ld, _lib.ptr(scale),
                                            _lib.stream_ptr(b.device)), "void_quant_i8_tensor")
    return q[:, :N], scale


def quantize_tensor(tensor: torch.Tensor, config: IntQuantConfig) -> Tuple[torch.Tensor, QuantizationParams]:
    """Quantise a tensor (void/int_quant.py:254-305).  PER_TENSOR and PER_BLOCK give one scale for
    the whole tensor (:271-276); PER_CHANNEL one per first-dimension slice (:273-274)."""
    _require_supported(config)
    _lib.require_cuda(tensor)
    shape = tuple(tensor.shape)
    if config.scale_mode == ScaleMode.PER_CHANNEL:
        flat = tensor.reshape(shape[0], -1)
        q_t, scale = quantize_cols_int8(flat.t())          # channels of `tensor` are columns of its transpose
        q = q_t.t().contiguous().reshape(shape)
        scale = scale.reshape((shape[0],) + (1,) * (len(shape) - 1))
    else:
        flat = tensor.reshape(1, -1) if tensor.dim() != 2 else tensor
        q, scale = _quantize_matrix_per_tensor(flat)
        q = q.contiguous().reshape(shape)
        scale = scale.reshape(())
    zero_point = torch.zeros_like(scale, dtype=torch.int8)
    return q, QuantizationParams(scale=scale, zero_point=zero_point, config=config, original_shape=shape)


def dequantize_tensor(quantized: torch.Tensor, params: QuantizationParams) -> torch.Tensor:
    """x = q * scale (void/int_quant.py:308-325, symmetric case)."""
    return quantized.float() * params.scale


def quantize_void_tensor(void_tensor, config: Optional[IntQuantConfig] = None) -> Int8VOIDTensor:
    """VOIDTensor -> Int8VOIDTensor with one symmetric scale per block (void/int_quant.py:328-388);
    the per-block Python loop of the reference (:363-369) is one kernel launch here."""
    if config is None:
        config = IntQuantConfig(format=IntFormat.INT8, symmetric=True, scale_mode=ScaleMode.PER_BLOCK)
    _require_supported(config)
    values = void_tensor.values
    _lib.require_cuda(values)
    lib = _lib.load()
    n_blocks = void_tensor.n_blocks
    tile_m, tile_k = void_tensor.tile_size
    dev = values.device
    if config.scale_mode == ScaleMode.PER_BLOCK:
        if (tile_m, tile_k) != (32, 32):
            raise NotImplementedError("void_b200 kernels are built for 32x32 tiles")
        vf = values.to(torch.float32).contiguous()
        q = torch.empty(n_blocks, tile_m, tile_k, dtype=torch.int8, device=dev)
        scales = torch.empty(n_blocks, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.void_quant_i8_tiles(_lib.ptr(vf), n_blocks, _lib.ptr(q), _lib.ptr(scales),
                                               _lib.stream_ptr(dev)), "void_quant_i8_tiles")
    else:
        q_flat, params = quantize_tensor(values.reshape(1, -1), IntQuantConfig(scale_mode=ScaleMode.PER_TENSOR))
        q = q_flat.reshape(n_blocks, tile_m, tile_k)
        scales = params.scale.reshape(1).expand(n_blocks).contiguous()
    return Int8VOIDTensor(values=q, scales=scales,
                          zero_points=torch.zeros(n_blocks, dtype=torch.int8, device=dev),
                          block_rows=void_tensor.block_rows.clone(), block_cols=void_tensor.block_cols.clone(),
                          shape=void_tensor.shape, tile_size=void_tensor.tile_size, n_blocks=n_blocks, config=config)


def dequantize_void_tensor(int8_tensor: Int8VOIDTensor):
    """Int8VOIDTensor -> fp32 VOIDTensor (void/int_quant.py:391-428; the reference version raises
    because it omits required VOIDTensor fields - they are filled in here)."""
    from .format import VOIDTensor, morton_encode_batch
    values = int8_tensor.values.float() * int8_tensor.scales.view(-1, 1, 1)
    codes = morton_encode_batch(int8_tensor.block_rows.cpu().numpy(), int8_tensor.block_cols.cpu().numpy())
    nbr, nbc = int8_tensor.block_grid
    return VOIDTensor(values=values, block_rows=int8_tensor.block_rows.clone(),
                      block_cols=int8_tensor.block_cols.clone(),
                      morton_codes=torch.as_tensor(codes.astype("int64"), device=values.device),
                      shape=int8_tensor.shape, tile_size=int8_tensor.tile_size,
                      nnz_original=int(torch.count_nonzero(values).item()), n_blocks=int8_tensor.n_blocks,
                      density=int8_tensor.n_blocks / max(nbr * nbc, 1), dtype=torch.float32)


def _resolve_b(b: torch.Tensor, b_scale):
    """(int8 B, scalar scale, per-column scale tensor or None) from the caller's B and b_scale."""
    if b.dtype != torch.int8:
        # a floating-point B is quantised with one scale for the whole tensor, void/int_quant.py:565-573
        q, scale = _quantize_matrix_per_tensor(b)
        return q, 1.0, scale.expand(b.shape[1])
    if b_scale is None:
        return b, 1.0, None
    if isinstance(b_scale, torch.Tensor):
        if b_scale.numel() == 1:
            return b, float(b_scale.item()), None
        if b_scale.numel() != b.shape[1]:
            raise ValueError("b_scale must be a scalar or hold one scale per column of B")
        return b, 1.0, b_scale.reshape(-1)
    return b, float(b_scale), None


def void_spmm_int8(a: Int8VOIDTensor, b: torch.Tensor, b_scale: Union[None, float, torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, *, out_dtype: Optional[torch.dtype] = None,
                   exact_scales: bool = False, acc_out: Optional[torch.Tensor] = None, activation: int = 0,
                   bias: Optional[torch.Tensor] = None, row_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """INT8 sparse-dense product C = dequant(A_q . B_q) (void/int_quant.py:543-612).

    a: Int8VOIDTensor [M, K];  b: int8 [K, N] (or floating point, then quantised per tensor);
    b_scale: scale of B - a float as in the reference, or a tensor [N] of per-column scales.
    Returns fp32 [M, N] unless ``out`` / ``out_dtype`` ask for fp16 / bf16.  ``acc_out`` (int32
    [n_block_rows*32, N]) receives the raw int32 accumulators.
    """
    M, K = a.shape
    N = b.shape[1]
    _lib.require_cuda(a.values, b, out)
    b_q, scalar, col_scale = _resolve_b(b, b_scale)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.float32, device=b.device)
    packed = a.packed()
    mode = _lib.SCALE_PER_TILE if exact_scales else _lib.SCALE_ROW_MEAN
    # every element of out is written by the kernel (zeros for empty tile rows), so the
    # reference's torch.zeros / out.zero_() (:580-583) has no counterpart here
    return _spmm.spmm(packed, b_q, out, scale_mode=mode, col_scale=col_scale, b_scale=scalar, bias=bias,
                      act=activation, acc_out=acc_out, row_bias=row_bias)


def get_quantization_error(original: torch.Tensor, config: IntQuantConfig) -> dict:
    """Error metrics of a quantise / dequantise round trip (void/int_quant.py:615-645)."""
    quantized, params = quantize_tensor(original, config)
    reconstructed = dequantize_tensor(quantized, params)
    abs_error = (original - reconstructed).abs()
    rel_error = abs_error / (original.abs() + 1e-8)
    return {
        "config": str(config),
        "mean_abs_error": abs_error.mean().item(),
        "max_abs_error": abs_error.max().item(),
        "mean_rel_error": rel_error.mean().item(),
        "max_rel_error": rel_error.max().item(),
        "snr_db": (10 * torch.log10(original.pow(2).mean() / abs_error.pow(2).mean())).item(),
        "compression_ratio": original.element_size() / (config.bits / 8),
    }


__all__ = [
    "IntFormat", "ScaleMode", "IntQuantConfig", "QuantizationParams", "Int8VOIDTensor", "quantize_tensor",
    "dequantize_tensor", "quantize_void_tensor", "dequantize_void_tensor", "void_spmm_int8",
    "get_quantization_error", "quantize_cols_int8",
]
