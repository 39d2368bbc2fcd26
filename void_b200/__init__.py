"""void_b200 - the quantized block-sparse SpMM path of VOID, rebuilt for B200 (sm_100a).

Same names as the reference's ``void`` package for everything on that path, so
``import void_b200 as void`` is a drop-in for: csr_to_void, void_spmm, quantize_void_tensor, void_spmm_int8,
void_tensor_to_fp8 / void_spmm_fp8, void_spmm_gelu, compute_stream_k_workload /
void_spmm_stream_k, shard_void_tensor / distributed_void_spmm.  All arithmetic runs in
hand-written CUDA behind a C ABI (include/void_b200.h); there is no Triton, no dispatch layer and
no CPU fallback.
"""
from .format import (VOIDTensor, csr_to_void, dense_to_void, morton_encode, morton_decode, morton_encode_batch,
                     void_from_block_mask, MIN_TENSOR_CORE_TILE)
from .int_quant import (IntFormat, ScaleMode, IntQuantConfig, QuantizationParams, Int8VOIDTensor, quantize_tensor,
                        dequantize_tensor, quantize_void_tensor, dequantize_void_tensor, void_spmm_int8,
                        get_quantization_error, quantize_cols_int8)
from .fp8 import (FP8Format, FP8Config, FP8ScalingInfo, FP8VOIDTensor, create_scaling_info, compute_amax,
                  quantize_to_fp8, dequantize_from_fp8, void_spmm_fp8, void_tensor_to_fp8, quantize_cols_fp8)
from .ops import void_spmm, void_spmv, void_linear
from .fusion import (ActivationType, FusedOpType, get_activation_code, void_spmm_gelu, void_spmm_relu, void_spmm_silu,
                     fused_sparse_mlp, FusedSparseOp, create_fused_spmm_gelu, create_fused_spmm_relu, create_sparse_mlp,
                     FusedSparseLinear)
from .autograd import VOIDSpMMFunction, VOIDLinearFunction, VOIDSpMM, SparseLinear, spmm_tile_grad, void_spmm_autograd
from .stream_k import (StreamKWorkload, compute_stream_k_workload, void_spmm_stream_k, analyze_workload_balance)
from .scheduler import WorkloadProfile, analyze_workload
from .distributed import (ShardingStrategy, DistributedVOIDTensor, shard_void_tensor, distributed_void_spmm,
                          broadcast_b, broadcast_spmm_overlapped)
from ._lib import VoidB200Error, check_device_status

__version__ = "0.1.0"
