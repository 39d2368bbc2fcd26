"""Generates the golden fixtures in this folder by running the reference implementation itself.

Run where the reference checkout is available (it is not needed to run the tests):

    REFERENCE_DIR=/path/to/void python tests/golden/make_golden.py

The reference's Triton kernels are executed on the CPU through the Triton interpreter
(TRITON_INTERPRET=1), so no GPU is needed.  Wrappers of the reference that insist on CUDA
tensors (FP8 SpMM, fused activation) are bypassed by launching their @triton.jit kernels with
the wrapper's own launch arithmetic (void/fp8.py:709-740, void/fusion.py:486-509).

Fixtures (all .npz, inputs included so that the tests do not depend on RNG stability):
  format_small.npz   csr_to_void + get_row_block_info on a ragged 203x170 matrix
  c1_plumbing.npz    the 512x512 / density 0.1 / N=128 plumbing workload: format fields, fp32 SpMM,
                     INT8 quantisation (A per block, B per column) and INT8 SpMM
  int8_small.npz     INT8 SpMM with empty tile rows, ragged M/K/N, scalar and per-column B scales
  fp8_small.npz      FP8 quantisation (tiles and columns) and the FP8 SpMM kernel
  gelu_small.npz     fused GELU epilogue of the activation kernel (with and without bias)
  streamk_small.npz  Stream-K worker tables for a power-law row-length distribution
  fp_small.npz       floating-point void_spmm (fp32 and fp16), void_spmv, fused GELU and the Stream-K
                     kernel on a ragged matrix with empty tile rows

  dense_small.npz    dense_to_void with and without a norm threshold on a ragged matrix

  backward_small.npz gradients of VOIDSpMMFunction (dL/dA_values per stored tile, dL/dB) for a given dL/dC

  shard_small.npz    shard_void_tensor for ROW_WISE, COLUMN_WISE and BLOCK_WISE at world sizes 1, 2, 3 and 8
                     (11 x 7 block grid: a remainder and ranks past the end): ranges, kept tiles in their
                     kept order, rebased block rows, local shape.  The reference function computes all of
                     that and then fails in its last statement, a VOIDTensor(...) call that omits three
                     required fields (void/distributed.py:179-186); the fixture is made with that one
                     constructor call given defaults for the three fields, everything before it unmodified.

A fixture whose arrays come out identical to the file already present is left untouched.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
sys.dont_write_bytecode = True
REF = os.environ.get("REFERENCE_DIR")
if not REF or not os.path.isdir(os.path.join(REF, "void")):
    raise SystemExit("set REFERENCE_DIR to a checkout of the reference (the folder that holds void/)")
sys.path.insert(0, REF)

import numpy as np  # noqa: E402
import scipy.sparse as sp  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402

import void  # noqa: E402
from void.fp8 import FP8Config, quantize_to_fp8, void_spmm_fp8_kernel, void_tensor_to_fp8, compute_amax  # noqa: E402
from void.fusion import (void_spmm_activation_kernel, void_spmm_activation_row_bias_kernel,  # noqa: E402
                         get_activation_code)
from void.int_quant import (IntQuantConfig, ScaleMode, quantize_tensor, quantize_void_tensor,  # noqa: E402
                            void_spmm_int8)
from void.ops import get_triton_dtype  # noqa: E402
from void.ops import void_spmv_kernel  # noqa: E402
from void.stream_k import compute_stream_k_workload, analyze_workload_balance, stream_k_spmm_kernel  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def save(name, **arrays):
    path = os.path.join(HERE, name)
    if os.path.exists(path):
        old = np.load(path)
        if set(old.files) == set(arrays) and all(
                old[k].dtype == np.asarray(v).dtype and np.array_equal(old[k], v, equal_nan=True)
                for k, v in arrays.items()):
            print("%-20s unchanged" % name)
            return
    np.savez_compressed(path, **arrays)
    print("%-20s %7.1f KB" % (name, os.path.getsize(path) / 1024))


def coo_inputs(m):
    c = m.tocoo()
    return dict(coo_row=c.row.astype(np.int32), coo_col=c.col.astype(np.int32), coo_data=c.data.astype(np.float32),
                shape=np.asarray(m.shape, dtype=np.int64))


def void_fields(vt, prefix=""):
    row_ptr, block_indices = vt.get_row_block_info()
    return {
        prefix + "values": vt.values.numpy(), prefix + "block_rows": vt.block_rows.numpy(),
        prefix + "block_cols": vt.block_cols.numpy(), prefix + "morton_codes": vt.morton_codes.numpy(),
        prefix + "row_ptr": row_ptr.numpy(), prefix + "block_indices": block_indices.numpy(),
        prefix + "meta": np.asarray([vt.n_blocks, vt.nnz_original], dtype=np.int64),
        prefix + "density": np.asarray([vt.density], dtype=np.float64),
    }


def per_column_int8(b):
    q, p = quantize_tensor(b.t().contiguous(), IntQuantConfig(scale_mode=ScaleMode.PER_CHANNEL))
    return q.t().contiguous(), p.scale.reshape(-1)


def ref_fp8_spmm(a8, b, out_dtype=torch.float32):
    """void_spmm_fp8 without its CUDA assert: same index build and launch as void/fp8.py:709-740."""
    M, K = a8.shape
    N = b.shape[1]
    tile_m, tile_k = a8.tile_size
    out = torch.zeros(M, N, dtype=out_dtype)
    nbr = (M + tile_m - 1) // tile_m
    row_counts = torch.zeros(nbr, dtype=torch.int32)
    row_counts.scatter_add_(0, a8.block_rows.long(), torch.ones_like(a8.block_rows))
    row_ptr = torch.zeros(nbr + 1, dtype=torch.int32)
    row_ptr[1:] = torch.cumsum(row_counts, dim=0)
    keys = a8.block_rows.long() * ((K + tile_k - 1) // tile_k) + a8.block_cols.long()
    block_indices = torch.argsort(keys).to(torch.int32)
    TILE_N = min(64, triton.next_power_of_2(N))
    scale_mode = 0 if a8.scaling_info.config.scale_mode == "per_tensor" else 1
    grid = (nbr, triton.cdiv(N, TILE_N))
    void_spmm_fp8_kernel[grid](
        a8.values_fp8, a8.scaling_info.scale, a8.block_rows, a8.block_cols, row_ptr, block_indices,
        b, out, M, N, K, a8.n_blocks, nbr, b.stride(0), b.stride(1), out.stride(0), out.stride(1),
        scale_mode, TILE_M=tile_m, TILE_K=tile_k, TILE_N=TILE_N, OUTPUT_DTYPE=get_triton_dtype(out_dtype))
    return out


def ref_gelu_spmm(vt, b, bias):
    """_void_spmm_activation(activation='gelu') without its CUDA assert, void/fusion.py:486-509."""
    M, K = vt.shape
    N = b.shape[1]
    out = torch.zeros(M, N, dtype=b.dtype)
    row_ptr, block_indices = vt.get_row_block_info()
    nbr = vt.block_grid[0]
    TILE_N = void.compute_optimal_tile_n(N)
    has_bias = 1 if bias is not None else 0
    bias_t = bias if bias is not None else torch.empty(1)
    grid = (nbr, triton.cdiv(N, TILE_N))
    void_spmm_activation_kernel[grid](
        vt.values, vt.block_rows, vt.block_cols, row_ptr, block_indices, b, bias_t, out,
        M, N, K, vt.n_blocks, nbr, b.stride(0), b.stride(1), out.stride(0), out.stride(1), has_bias,
        TILE_M=vt.tile_size[0], TILE_K=vt.tile_size[1], TILE_N=TILE_N, ACTIVATION=2,
        OUTPUT_DTYPE=get_triton_dtype(b.dtype))
    return out


def ref_row_bias_spmm(vt, b, bias, activation):
    """_void_spmm_activation_row_bias without its CUDA assert, void/fusion.py:352-377."""
    M, K = vt.shape
    N = b.shape[1]
    b = b.contiguous()
    out = torch.zeros(M, N, dtype=b.dtype)
    row_ptr, block_indices = vt.get_row_block_info()
    nbr = vt.block_grid[0]
    TILE_N = void.compute_optimal_tile_n(N)
    has_bias = 1 if bias is not None else 0
    bias_t = bias.contiguous() if bias is not None else torch.empty(1)
    grid = (nbr, triton.cdiv(N, TILE_N))
    void_spmm_activation_row_bias_kernel[grid](
        vt.values, vt.block_rows, vt.block_cols, row_ptr, block_indices, b, bias_t, out,
        M, N, K, vt.n_blocks, nbr, b.stride(0), b.stride(1), out.stride(0), out.stride(1), has_bias,
        TILE_M=vt.tile_size[0], TILE_K=vt.tile_size[1], TILE_N=TILE_N,
        ACTIVATION=get_activation_code(activation), OUTPUT_DTYPE=get_triton_dtype(b.dtype))
    return out


def ref_spmv(vt, x):
    """void_spmv without its CUDA assert, void/ops.py:320-347."""
    out = torch.zeros(vt.shape[0], dtype=x.dtype)
    row_ptr, block_indices = vt.get_row_block_info()
    nbr = vt.block_grid[0]
    void_spmv_kernel[(nbr,)](vt.values, vt.block_rows, vt.block_cols, row_ptr, block_indices, x, out,
                             vt.shape[0], vt.shape[1], vt.n_blocks, nbr, TILE_M=vt.tile_size[0],
                             TILE_K=vt.tile_size[1], OUTPUT_DTYPE=get_triton_dtype(x.dtype))
    return out


def ref_stream_k(vt, b, workload):
    """void_spmm_stream_k without its CUDA assert, void/stream_k.py:262-299."""
    M, K = vt.shape
    N = b.shape[1]
    tile_m, tile_k = vt.tile_size
    out = torch.zeros(M, N, dtype=b.dtype)
    _, block_indices = vt.get_row_block_info()
    locks = torch.zeros(((M + tile_m - 1) // tile_m) * ((N + 63) // 64), dtype=torch.int32)
    TILE_N = min(64, triton.next_power_of_2(N))
    grid = (workload.n_workers, triton.cdiv(N, TILE_N))
    stream_k_spmm_kernel[grid](
        vt.values, vt.block_cols, block_indices, workload.worker_rows, workload.worker_block_start,
        workload.worker_block_end, workload.worker_needs_atomic, b, out, locks, M, N, K, workload.n_workers,
        b.stride(0), b.stride(1), out.stride(0), out.stride(1), TILE_M=tile_m, TILE_K=tile_k, TILE_N=TILE_N,
        OUTPUT_DTYPE=get_triton_dtype(b.dtype))
    return out


def block_sparse_csr(rng, nbr, nbc, density, M=None, K=None, empty_rows=()):
    """Random block mask -> CSR with dense N(0,1) tiles (rows/cols beyond M/K dropped)."""
    M = M or nbr * 32
    K = K or nbc * 32
    mask = rng.random((nbr, nbc)) < density
    for r in empty_rows:
        mask[r] = False
    dense = np.zeros((nbr * 32, nbc * 32), dtype=np.float32)
    for r, c in zip(*np.nonzero(mask)):
        dense[r * 32:(r + 1) * 32, c * 32:(c + 1) * 32] = rng.standard_normal((32, 32)).astype(np.float32)
    return sp.csr_matrix(dense[:M, :K])


def main():
    # ---------------------------------------------------------------- format_small
    rng = np.random.default_rng(11)
    m = sp.random(203, 170, density=0.03, format="csr", dtype=np.float32, random_state=np.random.RandomState(5))
    m = m.tolil()
    m[40, 77] = 0.0          # stays a zero in the tile ...
    m = m.tocsr()
    m.data[3] = 0.0          # ... while an explicit stored zero still activates its tile
    vt = void.csr_to_void(m, tile_size=32)
    save("format_small.npz", **coo_inputs(m), **void_fields(vt))

    # ---------------------------------------------------------------- c1_plumbing
    np.random.seed(0)
    a = sp.random(512, 512, density=0.1, format="csr", dtype=np.float32)
    vt = void.csr_to_void(a, tile_size=32)
    torch.manual_seed(0)
    b = torch.randn(512, 128)
    c_fp32 = void.void_spmm(vt, b)
    q = quantize_void_tensor(vt)
    bq, bscale = per_column_int8(b)
    c_int8 = void_spmm_int8(q, bq, 1.0) * bscale[None, :]
    f = void_fields(vt)
    del f["values"]          # reproducible from the COO inputs; keeps the fixture small
    save("c1_plumbing.npz", **coo_inputs(a), b=b.numpy(), **f, c_fp32=c_fp32.numpy(),
         a_q=q.values.numpy(), a_scales=q.scales.numpy(), b_q=bq.numpy(), b_scales=bscale.numpy(),
         c_int8=c_int8.numpy())

    # ---------------------------------------------------------------- int8_small
    m = block_sparse_csr(rng, 7, 9, 0.45, M=200, K=270, empty_rows=(2, 5))
    vt = void.csr_to_void(m, tile_size=32)
    q = quantize_void_tensor(vt)
    b = torch.from_numpy(rng.standard_normal((270, 80)).astype(np.float32))
    bq, bscale = per_column_int8(b)
    c_unit = void_spmm_int8(q, bq, 1.0)
    c_scalar = void_spmm_int8(q, bq, 0.0371)
    c_float_b = void_spmm_int8(q, b)            # B quantised per tensor inside the wrapper
    save("int8_small.npz", **coo_inputs(m), b=b.numpy(), a_q=q.values.numpy(), a_scales=q.scales.numpy(),
         block_rows=q.block_rows.numpy(), block_cols=q.block_cols.numpy(), b_q=bq.numpy(),
         b_scales=bscale.numpy(), c_unit=c_unit.numpy(), c_scalar=c_scalar.numpy(),
         b_scalar=np.asarray([0.0371], dtype=np.float32), c_float_b=c_float_b.numpy())

    # ---------------------------------------------------------------- fp8_small
    m = block_sparse_csr(rng, 6, 8, 0.5, M=180, K=250, empty_rows=(1,))
    vt = void.csr_to_void(m, tile_size=32)
    a8 = void_tensor_to_fp8(vt, format="e4m3", scale_mode="per_block")
    a8t = void_tensor_to_fp8(vt, format="e4m3", scale_mode="per_tensor")
    b = torch.from_numpy(rng.standard_normal((250, 96)).astype(np.float32))
    b8, binfo = quantize_to_fp8(b.t().contiguous(), FP8Config(scale_mode="per_row"))
    b_deq = (b8.float() * binfo.scale[:, None]).t().contiguous()
    c_block = ref_fp8_spmm(a8, b_deq)
    c_block_rawb = ref_fp8_spmm(a8, b8.float().t().contiguous())      # unit B scales (epilogue check)
    c_tensor = ref_fp8_spmm(a8t, b_deq)
    c_f16 = ref_fp8_spmm(a8, b_deq, torch.float16)
    c_floatb = ref_fp8_spmm(a8, b)                # B given in floating point: used as it is
    kat = torch.tensor([[[1.0, 2.0], [3.0, 4.0]], [[5.0, 6.0], [7.0, 8.0]]])
    save("fp8_small.npz", **coo_inputs(m), b=b.numpy(), block_rows=a8.block_rows.numpy(),
         block_cols=a8.block_cols.numpy(), a_fp8=a8.values_fp8.view(torch.uint8).numpy(),
         a_scale=a8.scaling_info.scale.numpy(), a_scale_inv=a8.scaling_info.scale_inv.numpy(),
         a_amax=a8.scaling_info.amax.numpy(), a_amax_history=a8.scaling_info.amax_history.numpy(),
         at_fp8=a8t.values_fp8.view(torch.uint8).numpy(), at_scale=a8t.scaling_info.scale.reshape(1).numpy(),
         b_fp8=b8.t().contiguous().view(torch.uint8).numpy(), b_scale=binfo.scale.numpy(),
         b_scale_inv=binfo.scale_inv.numpy(), c_block=c_block.numpy(), c_block_rawb=c_block_rawb.numpy(),
         c_tensor=c_tensor.numpy(), c_f16=c_f16.float().numpy(), c_floatb=c_floatb.numpy(),
         kat_amax_tensor=compute_amax(kat, "per_tensor").reshape(1).numpy(),
         kat_amax_block=compute_amax(kat, "per_block").numpy())

    # ---------------------------------------------------------------- gelu_small
    m = block_sparse_csr(rng, 4, 5, 0.6, M=128, K=160)
    vt = void.csr_to_void(m, tile_size=32)
    b = torch.from_numpy(rng.standard_normal((160, 64)).astype(np.float32))
    bias = torch.from_numpy(rng.standard_normal(64).astype(np.float32))
    pre = void.void_spmm(vt, b)
    save("gelu_small.npz", pre=pre.numpy(), bias=bias.numpy(), post=ref_gelu_spmm(vt, b, None).numpy(),
         post_bias=ref_gelu_spmm(vt, b, bias).numpy())

    # ---------------------------------------------------------------- streamk_small
    z = np.minimum(rng.zipf(1.5, 96), 200)
    z[rng.random(96) < 0.1] = 0
    nbc = 256
    rows = np.repeat(np.arange(96), z)
    cols = np.concatenate([rng.choice(nbc, int(c), replace=False) for c in z]) if z.sum() else np.zeros(0, int)
    n = len(rows)
    mort = np.argsort(void.format.morton_encode_batch(rows, cols))
    vt = void.VOIDTensor(values=torch.zeros(n, 32, 32), block_rows=torch.tensor(rows[mort], dtype=torch.int32),
                         block_cols=torch.tensor(cols[mort], dtype=torch.int32),
                         morton_codes=torch.zeros(n, dtype=torch.int64), shape=(96 * 32, nbc * 32),
                         tile_size=(32, 32), nnz_original=n * 1024, n_blocks=n, density=n / (96 * nbc))
    out = {"block_rows": rows[mort].astype(np.int32), "block_cols": cols[mort].astype(np.int32),
           "grid": np.asarray([96, nbc], dtype=np.int64)}
    for tag, kw in (("default", {}), ("w64", {"n_workers": 64}), ("w300_m4", {"n_workers": 300, "max_work_per_worker": 4}),
                    ("w7", {"n_workers": 7})):
        w = compute_stream_k_workload(vt, **kw)
        out[tag + "_rows"] = w.worker_rows.numpy()
        out[tag + "_start"] = w.worker_block_start.numpy()
        out[tag + "_end"] = w.worker_block_end.numpy()
        out[tag + "_atomic"] = w.worker_needs_atomic.numpy()
        out[tag + "_meta"] = np.asarray([w.n_workers, w.total_work, kw.get("n_workers", -1),
                                         kw.get("max_work_per_worker", 16)], dtype=np.int64)
    bal = analyze_workload_balance(vt)
    out["balance"] = np.asarray([bal["n_rows"], bal["n_nonempty_rows"], bal["min_blocks_per_row"],
                                 bal["max_blocks_per_row"], bal["mean_blocks_per_row"], bal["std_blocks_per_row"],
                                 bal["imbalance_ratio"], bal["coefficient_of_variation"]], dtype=np.float64)
    save("streamk_small.npz", **out)

    # ---------------------------------------------------------------- fp_small
    rng = np.random.default_rng(23)
    m = block_sparse_csr(rng, 7, 9, 0.45, M=200, K=270, empty_rows=(1, 4))
    vt = void.csr_to_void(m, tile_size=32)
    b = torch.from_numpy(rng.standard_normal((270, 80)).astype(np.float32))
    bias = torch.from_numpy(rng.standard_normal(80).astype(np.float32))
    x = torch.from_numpy(rng.standard_normal(270).astype(np.float32))
    wl = compute_stream_k_workload(vt, n_workers=12, max_work_per_worker=2)
    assert wl.worker_needs_atomic.any()
    # two-layer MLP y = W2 @ gelu(W1 @ x^T + b1) + b2 (fused_sparse_mlp, void/fusion.py:557-602) on x = b^T
    m2 = block_sparse_csr(rng, 3, 7, 0.6, M=70, K=200)
    w2 = void.csr_to_void(m2, tile_size=32)
    bias1 = torch.from_numpy(rng.standard_normal(200).astype(np.float32))
    bias2 = torch.from_numpy(rng.standard_normal(70).astype(np.float32))
    hidden = ref_row_bias_spmm(vt, b, bias1, "gelu")
    mlp = ref_row_bias_spmm(w2, hidden, bias2, "none").T.contiguous()
    w2c = m2.tocoo()
    save("fp_small.npz", **coo_inputs(m), w2_row=w2c.row.astype(np.int32), w2_col=w2c.col.astype(np.int32),
         w2_data=w2c.data.astype(np.float32), bias1=bias1.numpy(), bias2=bias2.numpy(),
         rowbias_gelu=hidden.numpy(), rowbias_silu=ref_row_bias_spmm(vt, b, bias1, "silu").numpy(), mlp=mlp.numpy(), b=b.numpy(), bias=bias.numpy(), x=x.numpy(),
         block_rows=vt.block_rows.numpy(), block_cols=vt.block_cols.numpy(),
         c_fp32=void.void_spmm(vt, b).numpy(),
         c_f16=void.void_spmm(vt.half(), b.half()).float().numpy(),
         y_spmv=ref_spmv(vt, x).numpy(),
         gelu=ref_gelu_spmm(vt, b, None).numpy(), gelu_bias=ref_gelu_spmm(vt, b, bias).numpy(),
         stream_k=ref_stream_k(vt, b, wl).numpy(),
         stream_k_meta=np.asarray([wl.n_workers, 12, 2], dtype=np.int64))

    # ---------------------------------------------------------------- dense_small
    rng = np.random.default_rng(31)
    dense = block_sparse_csr(rng, 5, 7, 0.5, M=150, K=210, empty_rows=(3,)).toarray()
    dense[64:96, 0:32] = 0.01 * rng.standard_normal((32, 32)).astype(np.float32)   # a tile with a small L1 norm
    dense[10, 200] = 3.0                                                            # a single entry in an edge tile
    out = {"matrix": dense}
    for tag, thr in (("t0", 0.0), ("t10", 10.0)):
        vt = void.dense_to_void(torch.from_numpy(dense), tile_size=32, threshold=thr)
        f = void_fields(vt, tag + "_")
        del f[tag + "_row_ptr"], f[tag + "_block_indices"]
        out.update(f)
        out[tag + "_threshold"] = np.asarray([thr], dtype=np.float32)
    empty = void.dense_to_void(torch.zeros(40, 50), tile_size=32)
    out["empty_meta"] = np.asarray([empty.n_blocks, empty.nnz_original], dtype=np.int64)
    save("dense_small.npz", **out)

    # ---------------------------------------------------------------- backward_small
    from void.autograd import VOIDSpMMFunction
    rng = np.random.default_rng(47)
    m = block_sparse_csr(rng, 6, 5, 0.5, M=180, K=150, empty_rows=(2,))
    vt = void.csr_to_void(m, tile_size=32)
    b = torch.from_numpy(rng.standard_normal((150, 72)).astype(np.float32)).requires_grad_(True)
    grad_c = torch.from_numpy(rng.standard_normal((180, 72)).astype(np.float32))
    vals = vt.values.clone().requires_grad_(True)
    c = VOIDSpMMFunction.apply(vals, vt.block_rows, vt.block_cols, vt.shape, vt.tile_size, vt.n_blocks, b)
    c.backward(grad_c)
    save("backward_small.npz", **coo_inputs(m), b=b.detach().numpy(), grad_c=grad_c.numpy(),
         block_rows=vt.block_rows.numpy(), block_cols=vt.block_cols.numpy(), c=c.detach().numpy(),
         grad_values=vals.grad.numpy(), grad_b=b.grad.numpy())

    # ---------------------------------------------------------------- shard_small
    import void.format as ref_format
    from void.distributed import ShardingStrategy, shard_void_tensor
    rng = np.random.default_rng(53)
    m = block_sparse_csr(rng, 11, 7, 0.45, M=11 * 32 - 9, K=7 * 32 - 5, empty_rows=(4,))
    vt = void.csr_to_void(m, tile_size=32)
    vt.values[:, 0, 0] = torch.arange(vt.n_blocks, dtype=vt.values.dtype)     # every tile carries its own position
    real_ctor = ref_format.VOIDTensor

    def ctor_with_defaults(**kw):     # the three fields the reference's call leaves out
        kw.setdefault("morton_codes", torch.zeros(0, dtype=torch.int64))
        kw.setdefault("nnz_original", 0)
        kw.setdefault("density", 0.0)
        return real_ctor(**kw)

    out = {"block_rows": vt.block_rows.numpy(), "block_cols": vt.block_cols.numpy(),
           "shape": np.asarray(vt.shape, dtype=np.int64), "worlds": np.asarray([1, 2, 3, 8], dtype=np.int64)}
    ref_format.VOIDTensor = ctor_with_defaults
    try:
        for strat in (ShardingStrategy.ROW_WISE, ShardingStrategy.COLUMN_WISE, ShardingStrategy.BLOCK_WISE):
            for world in (1, 2, 3, 8):
                for rank in range(world):
                    d = shard_void_tensor(vt, strat, world, rank)
                    lt = d.local_tensor
                    tag = "%s_w%d_r%d_" % (strat.value, world, rank)
                    out[tag + "ids"] = lt.values[:, 0, 0].numpy().astype(np.int64)
                    out[tag + "rows"] = lt.block_rows.numpy().astype(np.int32)
                    out[tag + "cols"] = lt.block_cols.numpy().astype(np.int32)
                    out[tag + "meta"] = np.asarray(list(d.local_row_range) + list(d.local_col_range) + list(lt.shape) +
                                                   [lt.n_blocks] + list(d.global_shape), dtype=np.int64)
    finally:
        ref_format.VOIDTensor = real_ctor
    save("shard_small.npz", **out)


if __name__ == "__main__":
    main()
