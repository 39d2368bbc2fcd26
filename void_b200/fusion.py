"""Fused SpMM + activation epilogues on B200.

Mirrors ActivationType / get_activation_code (void/fusion.py:21-32, :77-91) and void_spmm_gelu
(:381-399).  GELU is the tanh form written with a sigmoid exactly as the reference kernel does
(:38-43): x * 0.5 * (1 + (2 * sigmoid(2u) - 1)), u = 0.7978845608 * (x + 0.044715 x^3); it is
applied to the dequantised fp32 accumulator (plus the column bias, :179-183) inside the SpMM
kernel's epilogue, before the fp16 / bf16 store.

The reference's void_spmm_gelu takes a floating-point VOIDTensor (TF32 product, result cast to B's
dtype, void/fusion.py:186-189); that form runs through void_spmm's kernel.  An Int8VOIDTensor or
FP8VOIDTensor selects the quantized kernels with the same epilogue.
"""
from enum import Enum
from typing import Optional, Union

import torch

from . import _lib
from .format import VOIDTensor
from .fp8 import FP8VOIDTensor, void_spmm_fp8
from .int_quant import Int8VOIDTensor, void_spmm_int8
from .ops import void_spmm


class ActivationType(Enum):
    NONE = "none"
    RELU = "relu"
    GELU = "gelu"
    SILU = "silu"
    TANH = "tanh"
    SIGMOID = "sigmoid"


def get_activation_code(activation: Union[str, ActivationType]) -> int:
    """Integer code of an activation name, same table as void/fusion.py:77-91."""
    if isinstance(activation, ActivationType):
        activation = activation.value
    codes = {"none": 0, "relu": 1, "gelu": 2, "silu": 3, "swish": 3, "tanh": 4, "sigmoid": 5}
    return codes.get(activation.lower(), 0)


def _void_spmm_activation(a, b, bias, out, activation: str, **kw) -> torch.Tensor:
    code = get_activation_code(activation)
    if code > _lib.ACT_SILU:
        raise NotImplementedError("activation %r is not fused on B200 (none, relu, gelu, silu are)" % activation)
    if isinstance(a, Int8VOIDTensor):
        out_dtype = kw.pop("out_dtype", None)
        return void_spmm_int8(a, b, kw.pop("b_scale", None), out, out_dtype=out_dtype, activation=code, bias=bias, **kw)
    if isinstance(a, FP8VOIDTensor):
        return void_spmm_fp8(a, b, kw.pop("output_dtype", torch.float16), out=out, activation=code, bias=bias, **kw)
    if isinstance(a, VOIDTensor):
        if kw:
            raise TypeError("unexpected keyword arguments for a floating-point VOIDTensor: %s" % sorted(kw))
        assert bias is None or bias.shape == (b.shape[1],), "bias must be a vector of N columns"   # void/fusion.py:452
        return void_spmm(a, b, out, activation=code, bias=bias)
    raise TypeError("void_spmm activation kernels take a VOIDTensor, Int8VOIDTensor or FP8VOIDTensor, got %s"
                    % type(a).__name__)


def void_spmm_gelu(a, b: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                   **kw) -> torch.Tensor:
    """C = GELU(A @ B + bias) in one kernel (void/fusion.py:381-399).  Keyword extensions for the
    quantized tensors: ``b_scale`` / ``out_dtype`` (INT8) or ``b_scale`` / ``output_dtype`` (FP8)."""
    return _void_spmm_activation(a, b, bias, out, "gelu", **kw)


def void_spmm_relu(a, b, bias=None, out=None, **kw) -> torch.Tensor:
    """C = ReLU(A @ B + bias) (void/fusion.py:402-420)."""
    return _void_spmm_activation(a, b, bias, out, "relu", **kw)


def void_spmm_silu(a, b, bias=None, out=None, **kw) -> torch.Tensor:
    """C = SiLU(A @ B + bias) (void/fusion.py:423-441)."""
    return _void_spmm_activation(a, b, bias, out, "silu", **kw)


__all__ = ["ActivationType", "get_activation_code", "void_spmm_gelu", "void_spmm_relu", "void_spmm_silu"]
