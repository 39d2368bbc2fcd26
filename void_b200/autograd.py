"""Differentiable SpMM on B200: VOIDSpMMFunction, VOIDSpMM and SparseLinear.

Mirrors void/autograd.py:99-347.  Forward is void_spmm (tensor cores, TF32 for fp32 operands).
Backward, as in the reference (:160-221):
    dL/dB        = A^T @ dL/dC        - void_spmm on the transposed tensor (tiles transposed, block rows and
                                        columns swapped, :178-191)
    dL/dA_values = dL/dC @ B^T        - for the stored tiles only: void_spmm_tile_grad, the tensor-core
                                        counterpart of void_spmm_backward_a_kernel (:14-96)
"""
from typing import Any, Optional, Tuple

import torch
from torch.autograd import Function

from . import _lib, _spmm, ops
from .format import VOIDTensor


# Tile index, backward work items and packed column list per sparsity structure.  The autograd function
# only sees bare tensors, and a layer's structure stays fixed while its values train, so the derived
# arrays are kept here, keyed by the identity of the index tensors (a handful of layers; oldest dropped).
_STRUCTURE = {}
_STRUCTURE_MAX = 64


def _structure(block_rows, block_cols, shape, n_blocks):
    key = (block_rows.data_ptr(), block_cols.data_ptr(), block_rows._version, block_cols._version, tuple(shape),
           n_blocks, str(block_rows.device))
    hit = _STRUCTURE.get(key)
    if hit is None:
        from .format import build_tile_index
        nbr, nbc = (shape[0] + 31) // 32, (shape[1] + 31) // 32
        row_ptr, block_indices = build_tile_index(block_rows, block_cols, nbr, nbc)
        tile_cols = block_cols.to(torch.int32)[block_indices.long()].contiguous()
        hit = (row_ptr, block_indices, tile_grad_items(row_ptr), tile_cols, block_rows, block_cols)  # keeps the keys alive
        if len(_STRUCTURE) >= _STRUCTURE_MAX:
            _STRUCTURE.pop(next(iter(_STRUCTURE)))
        _STRUCTURE[key] = hit
    return hit


def _bare_void(values, block_rows, block_cols, shape, tile_size, n_blocks) -> VOIDTensor:
    """VOIDTensor over bare tensors (no Morton codes), with the cached tile index of its structure attached."""
    v = VOIDTensor(values=values, block_rows=block_rows, block_cols=block_cols,
                   morton_codes=torch.empty(0, dtype=torch.int64, device=values.device), shape=tuple(shape),
                   tile_size=tuple(tile_size), nnz_original=0, n_blocks=n_blocks, density=0.0, dtype=values.dtype)
    if values.is_cuda and tuple(tile_size) == (32, 32):
        st = _structure(block_rows, block_cols, shape, n_blocks)
        v._row_ptr_cache, v._block_indices_cache = st[0], st[1]
    return v


def tile_grad_items(row_ptr: torch.Tensor) -> torch.Tensor:
    """Work items of void_spmm_tile_grad: every tile row cut into groups of up to four consecutive packed
    tiles -> int32 [n_items, 4] = (tile row, first packed tile, tile count, 0).  Depends on A's structure only."""
    rp = row_ptr.to(torch.int64)
    cnt = rp[1:] - rp[:-1]
    groups = (cnt + 3) // 4
    total = int(groups.sum().item())
    dev = row_ptr.device
    if total == 0:
        return torch.zeros(0, 4, dtype=torch.int32, device=dev)
    rows = torch.repeat_interleave(torch.arange(cnt.numel(), device=dev), groups)
    first = torch.cumsum(groups, 0) - groups
    within = torch.arange(total, device=dev) - first[rows]
    t0 = rp[rows] + 4 * within
    n = torch.minimum(torch.full_like(t0, 4), rp[rows + 1] - t0)
    return torch.stack([rows, t0, n, torch.zeros_like(n)], dim=1).to(torch.int32).contiguous()


def spmm_tile_grad(a: VOIDTensor, grad_output: torch.Tensor, b: torch.Tensor,
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """dL/dA_values [n_blocks, 32, 32] for C = A @ B given dL/dC (void/autograd.py:196-219), in A's tile order."""
    _lib.require_cuda(a.values, grad_output, b)
    if tuple(a.tile_size) != (32, 32):
        raise NotImplementedError("void_b200 kernels are built for 32x32 tiles, got tile_size=%s" % (a.tile_size,))
    M, K = a.shape
    N = b.shape[1]
    assert grad_output.shape == (M, N) and b.shape[0] == K
    out_dtype = out_dtype or a.values.dtype
    dev = b.device
    grad = torch.zeros(a.n_blocks, 32, 32, dtype=out_dtype, device=dev)     # torch.zeros_like(a_values), :198
    if a.n_blocks == 0 or N == 0:
        return grad
    dt = grad_output.dtype if (grad_output.dtype == b.dtype and b.dtype in (torch.float16, torch.bfloat16)) \
        else torch.float32
    kind = _lib.FP_KIND[dt]
    g = _spmm.prepare_b(grad_output.to(dt), dt.itemsize)
    bb = _spmm.prepare_b(b.to(dt), dt.itemsize)
    _, block_indices, items, tile_cols = _structure(a.block_rows, a.block_cols, a.shape, a.n_blocks)[:4]
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.void_spmm_tile_grad(_lib.ptr(g), g.stride(0) * dt.itemsize, _lib.ptr(bb), bb.stride(0) * dt.itemsize,
                                           M, K, N, kind, _lib.ptr(items), items.shape[0], _lib.ptr(tile_cols),
                                           _lib.ptr(block_indices), _lib.ptr(grad), _lib.OUT_DTYPE_CODE[out_dtype],
                                           _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)), "void_spmm_tile_grad")
    return grad


class VOIDSpMMFunction(Function):
    """C = A @ B with gradients for A's stored tiles and for B (void/autograd.py:99-221)."""

    @staticmethod
    def forward(ctx: Any, a_values, a_block_rows, a_block_cols, a_shape: Tuple[int, int], a_tile_size: Tuple[int, int],
                a_n_blocks: int, b: torch.Tensor) -> torch.Tensor:
        a = _bare_void(a_values.detach(), a_block_rows, a_block_cols, a_shape, a_tile_size, a_n_blocks)
        c = ops.void_spmm(a, b.detach())
        ctx.save_for_backward(a_values, a_block_rows, a_block_cols, b)
        ctx.a_shape, ctx.a_tile_size, ctx.a_n_blocks = tuple(a_shape), tuple(a_tile_size), a_n_blocks
        return c

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor):
        a_values, a_block_rows, a_block_cols, b = ctx.saved_tensors
        M, K = ctx.a_shape
        grad_a_values = grad_b = None
        grad_output = grad_output.contiguous()
        if ctx.needs_input_grad[6]:
            a_t = _bare_void(a_values.detach().permute(0, 2, 1).contiguous(), a_block_cols, a_block_rows, (K, M),
                             ctx.a_tile_size[::-1], ctx.a_n_blocks)
            grad_b = ops.void_spmm(a_t, grad_output.to(b.dtype)) if ctx.a_n_blocks else torch.zeros_like(b)
        if ctx.needs_input_grad[0]:
            a = _bare_void(a_values.detach(), a_block_rows, a_block_cols, ctx.a_shape, ctx.a_tile_size, ctx.a_n_blocks)
            grad_a_values = spmm_tile_grad(a, grad_output, b.detach())
        return grad_a_values, None, None, None, None, None, grad_b


class VOIDLinearFunction(Function):
    """y = x @ A^T (+ bias) for x [batch, in]: the linear layer on activations as they lie in memory
    (ops.void_linear), differentiable in A's stored tiles, x and the bias.
        dL/dx        = dL/dy @ A          - void_linear with the transposed tensor
        dL/dA_values = (dL/dy)^T @ x      - for the stored tiles only (void_spmm_tile_grad; its operands need
                                            the batch index contiguous, so dL/dy and x are transposed here)
        dL/dbias     = column sums of dL/dy
    The reference's SparseLinear computes (A @ x^T)^T through VOIDSpMMFunction and adds the bias as a
    separate op (void/autograd.py:320-344)."""

    @staticmethod
    def forward(ctx: Any, a_values, a_block_rows, a_block_cols, a_shape, a_tile_size, a_n_blocks: int, x, bias):
        a = _bare_void(a_values.detach(), a_block_rows, a_block_cols, a_shape, a_tile_size, a_n_blocks)
        y = ops.void_linear(a, x.detach(), None if bias is None else bias.detach())
        ctx.save_for_backward(a_values, a_block_rows, a_block_cols, x)
        ctx.a_shape, ctx.a_tile_size, ctx.a_n_blocks = tuple(a_shape), tuple(a_tile_size), a_n_blocks
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor):
        a_values, a_block_rows, a_block_cols, x = ctx.saved_tensors
        M, K = ctx.a_shape
        grad_output = grad_output.contiguous()
        grad_a_values = grad_x = grad_bias = None
        if ctx.needs_input_grad[6]:
            a_t = _bare_void(a_values.detach().permute(0, 2, 1).contiguous(), a_block_cols, a_block_rows, (K, M),
                             ctx.a_tile_size[::-1], ctx.a_n_blocks)
            grad_x = ops.void_linear(a_t, grad_output.to(x.dtype)) if ctx.a_n_blocks else torch.zeros_like(x)
        if ctx.needs_input_grad[0]:
            a = _bare_void(a_values.detach(), a_block_rows, a_block_cols, ctx.a_shape, ctx.a_tile_size, ctx.a_n_blocks)
            grad_a_values = spmm_tile_grad(a, grad_output.T.contiguous(), x.detach().T.contiguous())
        if ctx.has_bias and ctx.needs_input_grad[7]:
            grad_bias = grad_output.sum(0)
        return grad_a_values, None, None, None, None, None, grad_x, grad_bias


class VOIDSpMM(torch.nn.Module):
    """A VOID matrix as a module with a differentiable y = A @ x (void/autograd.py:224-291)."""

    def __init__(self, void_tensor: VOIDTensor, requires_grad: bool = True):
        super().__init__()
        if requires_grad:
            self.values = torch.nn.Parameter(void_tensor.values.clone())
        else:
            self.register_buffer("values", void_tensor.values.clone())
        self.register_buffer("block_rows", void_tensor.block_rows)
        self.register_buffer("block_cols", void_tensor.block_cols)
        self.shape, self.tile_size, self.n_blocks = void_tensor.shape, void_tensor.tile_size, void_tensor.n_blocks

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        squeeze = x.dim() == 1
        if squeeze:
            x = x.unsqueeze(1)
        y = VOIDSpMMFunction.apply(self.values, self.block_rows, self.block_cols, self.shape, self.tile_size,
                                   self.n_blocks, x)
        return y.squeeze(1) if squeeze else y

    def get_void_tensor(self) -> VOIDTensor:
        return _bare_void(self.values.data, self.block_rows, self.block_cols, self.shape, self.tile_size, self.n_blocks)


class SparseLinear(torch.nn.Module):
    """nn.Linear with a VOID weight: y = x W^T + b (void/autograd.py:294-347)."""

    def __init__(self, in_features: int, out_features: int, void_tensor: VOIDTensor, bias: bool = True,
                 dtype: Optional[torch.dtype] = None):
        super().__init__()
        assert void_tensor.shape == (out_features, in_features)
        self.in_features, self.out_features = in_features, out_features
        self.sparse_weight = VOIDSpMM(void_tensor, requires_grad=True)
        dtype = dtype or void_tensor.dtype
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=void_tensor.values.device))
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        input_shape = x.shape
        x_flat = x.reshape(-1, self.in_features)
        w = self.sparse_weight
        y = VOIDLinearFunction.apply(w.values, w.block_rows, w.block_cols, w.shape, w.tile_size, w.n_blocks, x_flat,
                                     self.bias)
        return y.reshape(input_shape[:-1] + (self.out_features,))

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


def void_spmm_autograd(a: VOIDTensor, b: torch.Tensor) -> torch.Tensor:
    """Differentiable C = A @ B for a VOIDTensor whose values (or B) require grad."""
    return VOIDSpMMFunction.apply(a.values, a.block_rows, a.block_cols, a.shape, a.tile_size, a.n_blocks, b)


__all__ = ["VOIDSpMMFunction", "VOIDLinearFunction", "VOIDSpMM", "SparseLinear", "spmm_tile_grad", "tile_grad_items", "void_spmm_autograd"]
