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
from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Union

import torch

from . import _lib
from .format import VOIDTensor
from .fp8 import FP8VOIDTensor, void_spmm_fp8
from .int_quant import Int8VOIDTensor, void_spmm_int8
from .ops import void_linear, void_spmm


class FusedOpType(Enum):
    """Fused operation kinds (void/fusion.py:14-21)."""
    SPMM_GELU = "spmm_gelu"
    SPMM_RELU = "spmm_relu"
    SPMM_SILU = "spmm_silu"
    SPMM_BIAS_GELU = "spmm_bias_gelu"
    SPMM_BIAS_RELU = "spmm_bias_relu"
    SPARSE_MLP = "sparse_mlp"


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


def _void_spmm_activation_row_bias(a, b: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor],
                                   activation: str, **kw) -> torch.Tensor:
    """C = activation(A @ B + bias[:, None]) in one kernel: the linear-layer form, bias per output row
    (void/fusion.py:307-378; kernel :201-304).  ``a`` may also be an Int8VOIDTensor (extension)."""
    code = get_activation_code(activation)
    if code > _lib.ACT_SILU:
        raise NotImplementedError("activation %r is not fused on B200 (none, relu, gelu, silu are)" % activation)
    assert b.dim() == 2
    assert a.shape[1] == b.shape[0]
    M = a.shape[0]
    if bias is not None:
        assert bias.shape == (M,), f"Row-wise bias must have shape ({M},), got {tuple(bias.shape)}"
    if isinstance(a, Int8VOIDTensor):
        return void_spmm_int8(a, b, kw.pop("b_scale", None), out, out_dtype=kw.pop("out_dtype", None), activation=code,
                              row_bias=bias, **kw)
    if kw:
        raise TypeError("unexpected keyword arguments for a floating-point VOIDTensor: %s" % sorted(kw))
    return void_spmm(a, b, out, activation=code, row_bias=bias)


def fused_sparse_mlp(x: torch.Tensor, w1: VOIDTensor, w2: VOIDTensor, activation: str = "gelu",
                     bias1: Optional[torch.Tensor] = None, bias2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = W2 @ activation(W1 @ x + b1) + b2 for x of shape [*, in_features] (void/fusion.py:557-602): two
    launches, each with its bias and activation fused.  Activations stay [batch, features] throughout
    (void_linear): none of the reference's three transposes is made."""
    code = get_activation_code(activation)
    if code > _lib.ACT_SILU:
        raise NotImplementedError("activation %r is not fused on B200 (none, relu, gelu, silu are)" % activation)
    input_shape = x.shape
    x_2d = x.reshape(-1, x.shape[-1])
    hidden = void_linear(w1, x_2d, bias1, code)
    out = void_linear(w2, hidden, bias2, 0)
    return out.reshape(input_shape[:-1] + (out.shape[-1],))


@dataclass
class FusedSparseOp:
    """A configured fused sparse operation (void/fusion.py:518-554)."""
    op_type: FusedOpType
    sparse_tensors: List[VOIDTensor]
    activation: Optional[str] = "gelu"
    biases: Optional[List[torch.Tensor]] = None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        first_bias = self.biases[0] if self.biases else None
        if self.op_type == FusedOpType.SPMM_GELU:
            return void_spmm_gelu(self.sparse_tensors[0], x, first_bias)
        if self.op_type == FusedOpType.SPMM_RELU:
            return void_spmm_relu(self.sparse_tensors[0], x, first_bias)
        if self.op_type == FusedOpType.SPMM_SILU:
            return void_spmm_silu(self.sparse_tensors[0], x, first_bias)
        if self.op_type == FusedOpType.SPARSE_MLP:
            return fused_sparse_mlp(x, self.sparse_tensors[0], self.sparse_tensors[1], activation=self.activation,
                                    bias1=first_bias,
                                    bias2=self.biases[1] if self.biases and len(self.biases) > 1 else None)
        raise ValueError(f"Unknown fused op type: {self.op_type}")


def create_fused_spmm_gelu(weight: VOIDTensor, bias: Optional[torch.Tensor] = None) -> FusedSparseOp:
    return FusedSparseOp(FusedOpType.SPMM_GELU, [weight], "gelu", [bias] if bias is not None else None)


def create_fused_spmm_relu(weight: VOIDTensor, bias: Optional[torch.Tensor] = None) -> FusedSparseOp:
    return FusedSparseOp(FusedOpType.SPMM_RELU, [weight], "relu", [bias] if bias is not None else None)


def create_sparse_mlp(w1: VOIDTensor, w2: VOIDTensor, activation: str = "gelu", bias1: Optional[torch.Tensor] = None,
                      bias2: Optional[torch.Tensor] = None) -> FusedSparseOp:
    """As void/fusion.py:730-753, including its packing of the biases that are present into one list."""
    biases = [b for b in (bias1, bias2) if b is not None]
    return FusedSparseOp(FusedOpType.SPARSE_MLP, [w1, w2], activation, biases if biases else None)


class FusedSparseLinear(torch.nn.Module):
    """y = activation(W @ x + b) with a VOID weight, one launch per call (void/fusion.py:756-836).
    Inference only: the weight tiles are a buffer and no backward is defined."""

    def __init__(self, in_features: int, out_features: int, void_tensor: VOIDTensor, activation: str = "gelu",
                 bias: bool = True):
        super().__init__()
        assert void_tensor.shape == (out_features, in_features)
        self.in_features, self.out_features, self.activation = in_features, out_features, activation
        self.register_buffer("values", void_tensor.values.clone())
        self.register_buffer("block_rows", void_tensor.block_rows)
        self.register_buffer("block_cols", void_tensor.block_cols)
        self.register_buffer("morton_codes", void_tensor.morton_codes)
        self.shape, self.tile_size, self.n_blocks = void_tensor.shape, void_tensor.tile_size, void_tensor.n_blocks
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(out_features, device=void_tensor.values.device))
        else:
            self.register_parameter("bias", None)
        self._void = None

    def get_void_tensor(self) -> VOIDTensor:
        """The VOIDTensor over the module's buffers; kept between calls so that its packed copy is reused
        (rebuilt when the buffers move or change)."""
        v = self._void
        if v is None or v.values.data_ptr() != self.values.data_ptr():
            v = self._void = VOIDTensor(values=self.values, block_rows=self.block_rows, block_cols=self.block_cols,
                                        morton_codes=self.morton_codes, shape=self.shape, tile_size=self.tile_size,
                                        nnz_original=0, n_blocks=self.n_blocks, density=0.0, dtype=self.values.dtype)
        return v

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        input_shape = x.shape
        x_flat = x.reshape(-1, self.in_features)
        bias = None if self.bias is None else self.bias.detach()
        code = get_activation_code(self.activation)
        if code > _lib.ACT_SILU:
            raise NotImplementedError("activation %r is not fused on B200" % self.activation)
        y = void_linear(self.get_void_tensor(), x_flat, bias, code)            # [batch, out], no transposes
        return y.reshape(input_shape[:-1] + (self.out_features,))

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"activation={self.activation}, bias={self.bias is not None}")


__all__ = ["ActivationType", "FusedOpType", "get_activation_code", "void_spmm_gelu", "void_spmm_relu", "void_spmm_silu",
           "fused_sparse_mlp", "FusedSparseOp", "create_fused_spmm_gelu", "create_fused_spmm_relu", "create_sparse_mlp",
           "FusedSparseLinear"]
