"""Floating-point SpMM / SpMV on B200: C = A @ B with A a VOIDTensor of fp32, fp16 or bf16 tiles.

Mirrors void_spmm (void/ops.py:148-217) and void_spmv (:286-349).  The reference kernel casts both
tiles to fp32 and calls tl.dot (:118-133), which multiplies in TF32 on a GPU and accumulates in
fp32; the result is stored in B's dtype (:183, :146).  Here the same pipeline as the quantized
kernels runs with tcgen05 kind::tf32 (fp32 operands; products in TF32, fp32 accumulation) or,
when A's tiles and B are both fp16 or both bf16, kind::f16 (exact products, fp32 accumulation).
Mixed dtypes are brought to fp32 like the reference's casts.
"""
from typing import Optional

import torch

from . import _lib, _spmm
from .format import VOIDTensor

_KIND_DTYPE = {_lib.KIND_F16: torch.float16, _lib.KIND_BF16: torch.bfloat16, _lib.KIND_TF32: torch.float32}


def product_kind(a: VOIDTensor, b: torch.Tensor) -> int:
    """Tensor-core kind for A's tiles and B: their common 16-bit type, else fp32 operands (TF32)."""
    if a.values.dtype == b.dtype and b.dtype in (torch.float16, torch.bfloat16):
        return _lib.FP_KIND[b.dtype]
    if not (a.values.dtype.is_floating_point and b.dtype.is_floating_point):
        raise _lib.VoidB200Error("void_spmm takes floating-point tiles and a floating-point B, got %s and %s"
                                 % (a.values.dtype, b.dtype))
    return _lib.KIND_TF32


def packed_fp(a: VOIDTensor, kind: int) -> _spmm.PackedTiles:
    """Packed copy of a floating VOIDTensor for ``kind`` (built once per kind, cached on the tensor)."""
    if tuple(a.tile_size) != (_spmm.TILE, _spmm.TILE):
        raise NotImplementedError("void_b200 kernels are built for 32x32 tiles, got tile_size=%s" % (a.tile_size,))
    cache = getattr(a, "_packed_fp_cache", None)
    if cache is None:
        cache = a._packed_fp_cache = {}
    key = (a.values.data_ptr(), a.values._version, a.block_rows.data_ptr(), a.block_cols.data_ptr(),
           str(a.values.device), tuple(a.shape))
    hit = cache.get(kind)
    if hit is not None and hit.key == key:
        return hit
    vals = a.values if a.values.dtype == _KIND_DTYPE[kind] else a.values.to(_KIND_DTYPE[kind])
    row_ptr, block_indices = a.get_row_block_info()
    p = _spmm._mark_ready(_spmm.pack(vals, None, a.block_rows, a.block_cols, a.shape, kind, row_ptr, block_indices))
    p.key = key
    cache[kind] = p
    a._plan_cache = {}
    return p


def void_spmm(a: VOIDTensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *, activation: int = 0,
              bias: Optional[torch.Tensor] = None, row_bias: Optional[torch.Tensor] = None, plan=None,
              acc_out: Optional[torch.Tensor] = None, worker_partials: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ B (void/ops.py:148-217); ``out`` defaults to a new [M, N] tensor of B's dtype.

    Keyword extensions: ``activation`` (code of get_activation_code: none, relu, gelu, silu) and a
    column ``bias`` [N] or a ``row_bias`` [M] fused into the epilogue; ``plan`` (a work plan of
    stream_k.stream_k_plan).
    """
    assert b.dim() == 2
    assert a.shape[1] == b.shape[0], f"Dimension mismatch: A is {a.shape}, B is {tuple(b.shape)}"
    _lib.require_cuda(a.values, b)
    M, _ = a.shape
    N = b.shape[1]
    if b.dtype not in _lib.OUT_DTYPE_CODE:
        raise _lib.VoidB200Error("void_spmm: B must be float32, float16 or bfloat16, got %s" % b.dtype)
    if out is None:
        out = torch.empty(M, N, dtype=b.dtype, device=b.device)
    if a.n_blocks == 0 and activation == 0 and bias is None and row_bias is None and plan is None \
            and acc_out is None and worker_partials is None:
        return out.zero_()      # nothing stored: zeros, whatever the tile size (void/ops.py:169-173)
    kind = product_kind(a, b)
    packed = packed_fp(a, kind)
    if b.dtype != _KIND_DTYPE[kind]:
        b = b.to(_KIND_DTYPE[kind])
    return _spmm.spmm(packed, b, out, scale_mode=_lib.SCALE_ROW_MEAN, use_row_scale=False, bias=bias, act=activation,
                      row_bias=row_bias, plan=plan, acc_out=acc_out, worker_partials=worker_partials)


def void_linear(a, x: torch.Tensor, bias: Optional[torch.Tensor] = None, activation: int = 0,
                out: Optional[torch.Tensor] = None, *, x_scale=None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = act(x @ A^T + bias) for activations x [batch, in] and a VOID weight A [out, in]: the linear layer
    without transposed copies.  The reference computes (A @ x^T)^T and so copies x^T and returns a strided
    view (void/fusion.py:586-598, :817-829; void/autograd.py:336); here the kernel reads x and writes y as
    they lie in memory.  ``a`` is a floating VOIDTensor (y in x's dtype) or an Int8VOIDTensor (x int8 with
    per-row scales ``x_scale`` [batch], or a float scalar; y fp32 unless ``out_dtype`` / ``out`` say otherwise).
    ``bias`` has one value per output feature."""
    from .int_quant import Int8VOIDTensor
    assert x.dim() == 2 and x.shape[1] == a.shape[1], f"Dimension mismatch: A is {a.shape}, x is {tuple(x.shape)}"
    _lib.require_cuda(a.values, x)
    M = a.shape[0]
    if bias is not None:
        assert bias.shape == (M,), f"bias must have shape ({M},), got {tuple(bias.shape)}"
    if isinstance(a, Int8VOIDTensor):
        if x.dtype != torch.int8:
            raise _lib.VoidB200Error("void_linear with an Int8VOIDTensor takes int8 activations, got %s" % x.dtype)
        scalar, col_scale = (1.0, x_scale) if isinstance(x_scale, torch.Tensor) else (1.0 if x_scale is None else float(x_scale), None)
        if out is None:
            out = torch.empty(x.shape[0], M, dtype=out_dtype or torch.float32, device=x.device)
        return _spmm.spmm(a.packed(), x, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=col_scale, b_scale=scalar,
                          act=activation, row_bias=bias, transposed=True)
    if x.dtype not in _lib.OUT_DTYPE_CODE:
        raise _lib.VoidB200Error("void_linear: x must be float32, float16 or bfloat16, got %s" % x.dtype)
    if out is None:
        out = torch.empty(x.shape[0], M, dtype=x.dtype, device=x.device)
    kind = product_kind(a, x)
    packed = packed_fp(a, kind)
    if x.dtype != _KIND_DTYPE[kind]:
        x = x.to(_KIND_DTYPE[kind])
    return _spmm.spmm(packed, x, out, scale_mode=_lib.SCALE_ROW_MEAN, use_row_scale=False, act=activation, row_bias=bias,
                      transposed=True)


def void_spmv(a: VOIDTensor, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = A @ x (void/ops.py:286-349): the one-column case of void_spmm."""
    squeeze_output = False
    if x.dim() == 2 and x.shape[1] == 1:
        x = x.squeeze(1)
        squeeze_output = True
    assert x.dim() == 1, "x must be 1D vector"
    assert a.shape[1] == x.shape[0], f"Dimension mismatch: A is {a.shape}, x is {tuple(x.shape)}"
    M = a.shape[0]
    if out is not None:
        assert out.shape == (M,)
    y = void_spmm(a, x.unsqueeze(1), None if out is None else out.unsqueeze(1))
    y = y.squeeze(1) if out is None else out
    return y.unsqueeze(1) if squeeze_output else y


__all__ = ["void_spmm", "void_spmv", "void_linear"]
