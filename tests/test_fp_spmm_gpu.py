"""GPU parity of the floating-point path (void_spmm, void_spmv, void_spmm_gelu and void_spmm_stream_k on
a floating VOIDTensor) against the CPU oracle and against outputs of the reference itself.

Bars: the reference's own, max|C - C_ref| / max|C_ref| < 1e-3 (tests/test_all_features.py:47-48, :155),
for fp32 operands multiplied as TF32; 16-bit operands multiply exactly and are held to the rounding of
the 16-bit result."""
import numpy as np
import pytest
import torch

import void_b200 as void
from void_b200 import stream_k, workloads
from conftest import coo_to_csr, load_golden, rel_err
from oracle import void_oracle as vo

pytestmark = pytest.mark.gpu
TF32_BAR = 1e-3


def _np(t):
    return t.detach().float().cpu().numpy()


def _oracle(a, b):
    return vo.spmm_fp(_np(a.values), _np(a.block_rows).astype(np.int32), _np(a.block_cols).astype(np.int32),
                      a.shape, _np(b))


def test_fp32_spmm_c1_vs_reference_output():
    g = load_golden("c1_plumbing.npz")
    a = void.csr_to_void(coo_to_csr(g), tile_size=32, device="cuda")
    b = torch.from_numpy(g["b"]).cuda()
    c = void.void_spmm(a, b)
    assert c.dtype == torch.float32 and c.shape == (512, 128)
    assert rel_err(_np(c), g["c_fp32"]) < TF32_BAR
    assert rel_err(_np(c), _oracle(a, b)) < TF32_BAR
    out = torch.full((512, 128), 7.0, device="cuda")
    assert void.void_spmm(a, b, out) is out and torch.equal(out, c)       # a given buffer is overwritten
    void.check_device_status()


def test_fp_small_all_entry_points_vs_reference_output():
    g = load_golden("fp_small.npz")
    a = void.csr_to_void(coo_to_csr(g), tile_size=32, device="cuda")
    b = torch.from_numpy(g["b"]).cuda()
    bias = torch.from_numpy(g["bias"]).cuda()
    c = void.void_spmm(a, b)                                               # ragged M, K, N; empty tile rows
    assert rel_err(_np(c), g["c_fp32"]) < TF32_BAR
    assert not c[32:64].any() and not c[128:160].any()
    y = void.void_spmv(a, torch.from_numpy(g["x"]).cuda())
    assert y.shape == (200,) and rel_err(_np(y), g["y_spmv"]) < TF32_BAR
    y2 = void.void_spmv(a, torch.from_numpy(g["x"]).cuda()[:, None])
    assert y2.shape == (200, 1) and torch.equal(y2[:, 0], y)
    assert rel_err(_np(void.void_spmm_gelu(a, b)), g["gelu"]) < TF32_BAR
    assert rel_err(_np(void.void_spmm_gelu(a, b, bias)), g["gelu_bias"]) < TF32_BAR
    relu = void.void_spmm_relu(a, b, bias)
    assert torch.equal(relu, torch.relu(void.void_spmm(a, b, bias=bias)))
    # fp16 tiles x fp16 B: exact products, fp32 sums, one rounding to fp16
    c16 = void.void_spmm(a.half(), b.half())
    assert c16.dtype == torch.float16 and rel_err(_np(c16), g["c_f16"]) < 1e-3
    # mixed dtypes go through fp32 like the reference's casts; the result takes B's dtype
    cm = void.void_spmm(a.half(), b)
    assert cm.dtype == torch.float32 and rel_err(_np(cm), _oracle(a.half(), b)) < TF32_BAR
    # Stream-K with the reference's table for (12 workers, at most 2 tiles each)
    wl = void.compute_stream_k_workload(a, n_workers=12, max_work_per_worker=2)
    assert wl.n_workers == int(g["stream_k_meta"][0]) and wl.worker_needs_atomic.any()
    for n_cta in (None, 3):
        for _ in range(2):                                                 # scratch is left clean between calls
            s = void.void_spmm_stream_k(a, b, wl, n_cta=n_cta)
            assert s.dtype == torch.float32 and rel_err(_np(s), g["stream_k"]) < TF32_BAR
            assert rel_err(_np(s), _np(c)) < 1e-6                          # same products, other summation order
    void.check_device_status()


def test_row_bias_mlp_and_linear_module_vs_reference_output():
    import scipy.sparse as sp
    g = load_golden("fp_small.npz")
    w1 = void.csr_to_void(coo_to_csr(g), tile_size=32, device="cuda")
    w2 = void.csr_to_void(sp.csr_matrix((g["w2_data"], (g["w2_row"], g["w2_col"])), shape=(70, 200)), tile_size=32,
                          device="cuda")
    b = torch.from_numpy(g["b"]).cuda()
    b1, b2 = torch.from_numpy(g["bias1"]).cuda(), torch.from_numpy(g["bias2"]).cuda()
    from void_b200.fusion import _void_spmm_activation_row_bias
    h = _void_spmm_activation_row_bias(w1, b, b1, None, "gelu")
    assert rel_err(_np(h), g["rowbias_gelu"]) < TF32_BAR
    assert rel_err(_np(_void_spmm_activation_row_bias(w1, b, b1, None, "silu")), g["rowbias_silu"]) < TF32_BAR
    x = b.T.contiguous()                                                    # [batch 80, in 270]
    y = void.fused_sparse_mlp(x, w1, w2, "gelu", b1, b2)
    assert y.shape == (80, 70) and rel_err(_np(y), g["mlp"]) < 2 * TF32_BAR  # two TF32 products in a row
    y3 = void.fused_sparse_mlp(x.reshape(4, 20, 270), w1, w2, "gelu", b1, b2)
    assert y3.shape == (4, 20, 70) and torch.equal(y3.reshape(80, 70), y)
    assert torch.equal(void.create_sparse_mlp(w1, w2, "gelu", b1, b2)(x), y)
    assert torch.equal(void.create_fused_spmm_gelu(w1)(b), void.void_spmm_gelu(w1, b))
    lin = void.FusedSparseLinear(270, 200, w1, activation="gelu", bias=True)
    with torch.no_grad():
        lin.bias.copy_(b1)
    assert torch.allclose(lin(x), h.T, rtol=1e-6, atol=1e-6) and "in_features=270" in repr(lin)
    assert lin(x).is_contiguous()
    with pytest.raises(AssertionError):
        _void_spmm_activation_row_bias(w1, b, b2, None, "gelu")            # wrong bias length
    # the same epilogue on the quantized kernel (extension): bias per row after dequantisation
    q = void.quantize_void_tensor(w1)
    bq, bs = void.quantize_cols_int8(b)
    pre = void.void_spmm_int8(q, bq, bs)
    got = _void_spmm_activation_row_bias(q, bq, b1, None, "relu", b_scale=bs)
    assert torch.allclose(got, torch.relu(pre + b1[:, None]), rtol=1e-6, atol=1e-6)
    void.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int8])
@pytest.mark.parametrize("batch", [1, 100, 128, 300])
def test_linear_without_transposes_exact_on_small_integers(dtype, batch):
    # y = x @ A^T with x [batch, in] and y [batch, out] as they lie in memory; small integers are exact in every
    # kind, so any slip in the K-major operand layout (swizzle span of 32 / 64 / 128 bytes) shows as a wrong integer
    mask = workloads.uniform_mask(7, 9, 0.5, seed=batch)
    mask[2] = False
    gen = torch.Generator().manual_seed(batch)
    tiles = torch.randint(-3, 4, (int(mask.sum()), 32, 32), generator=gen).float()
    a = void.void_from_block_mask(mask, tiles, shape=(200, 270), device="cuda")     # ragged out / in features
    x = torch.randint(-3, 4, (batch, 270), generator=gen).float().cuda()
    ref = x @ a.to_dense().T
    bias = torch.randint(-5, 6, (200,), generator=gen).float().cuda()
    if dtype == torch.int8:
        q = void.quantize_void_tensor(a)
        xs = torch.rand(batch, generator=gen).cuda() + 0.5
        y = void.void_linear(q, x.to(torch.int8), bias, 1, x_scale=xs)
        ref_q = void.void_spmm_int8(q, x.to(torch.int8).T.contiguous(), xs, bias=None, row_bias=bias, activation=1).T
        assert y.shape == (batch, 200) and y.dtype == torch.float32 and torch.equal(y, ref_q)
    else:
        y = void.void_linear(a.to_dtype(dtype), x.to(dtype), out=torch.empty(batch, 200, device="cuda"))
        assert torch.equal(y, ref)
        yb = void.void_linear(a.to_dtype(dtype), x.to(dtype), bias, 1)
        assert yb.dtype == dtype and torch.equal(yb.float(), torch.relu(ref + bias[None, :]).to(dtype).float())
        wide = torch.full((batch, 264), 9.0, device="cuda")                         # output rows with a larger pitch
        void.void_linear(a.to_dtype(dtype), x.to(dtype), out=wide[:, :200])
        assert torch.equal(wide[:, :200], ref) and bool((wide[:, 200:] == 9.0).all())
    void.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [32, 96, 200, 512])
def test_fp_spmm_shapes_and_dtypes(dtype, n):
    mask = workloads.uniform_mask(24, 40, 0.75, seed=n)
    mask[3] = False
    w = workloads.block_sparse(mask, n, seed=5)
    a = w.a.to_dtype(dtype)
    b = w.b.to(dtype)
    c = void.void_spmm(a, b)
    ref = _oracle(a, b)
    assert c.dtype == dtype
    if dtype == torch.float32:
        assert rel_err(_np(c), ref) < TF32_BAR
    else:
        # exact products and fp32 sums: only the final rounding to the 16-bit type separates the two
        eps = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
        assert np.abs(_np(c) - ref).max() <= eps * np.abs(ref).max() * 1.01
    void.check_device_status()


def test_fp32_products_are_exact_for_tf32_representable_inputs():
    # integers below 2^10 survive the TF32 rounding and their sums stay exact in fp32: any slip in the
    # operand layouts (tile packing, panel swizzle, k order) would show as a wrong integer
    mask = workloads.uniform_mask(8, 12, 0.5, seed=1)
    gen = torch.Generator().manual_seed(2)
    tiles = torch.randint(-7, 8, (int(mask.sum()), 32, 32), generator=gen).float()
    a = void.void_from_block_mask(mask, tiles, device="cuda")
    b = torch.randint(-7, 8, (12 * 32, 160), generator=gen).float().cuda()
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        c = void.void_spmm(a.to_dtype(dt), b.to(dt), torch.empty(256, 160, device="cuda"))
        assert np.array_equal(_np(c), _oracle(a, b)), dt


def test_fp_stream_k_power_law_rows():
    mask = workloads.zipf_mask(96, 256, 1.5, 200, 12.0, 7)
    w = workloads.block_sparse(mask, 192, 7)
    c = void.void_spmm(w.a, w.b)
    assert rel_err(_np(c), _oracle(w.a, w.b)) < TF32_BAR
    wl = void.compute_stream_k_workload(w.a)
    plan = stream_k.stream_k_plan(w.a, 192, wl)
    assert plan.n_counters > 0                                             # some rows are split between CTAs
    for _ in range(3):
        s = void.void_spmm_stream_k(w.a, w.b, wl)
        assert rel_err(_np(s), _np(c)) < 1e-5
    g = void.void_spmm_stream_k(w.a, w.b, activation=2)
    assert rel_err(_np(g), vo.gelu_tanh_sigmoid(_np(c))) < 1e-5
    void.check_device_status()


def test_fp_spmm_refuses_what_it_does_not_do():
    mask = workloads.uniform_mask(4, 4, 0.5, seed=0)
    w = workloads.block_sparse(mask, 64, 0)
    with pytest.raises(void.VoidB200Error):
        void.void_spmm(w.a, w.b.double())
    with pytest.raises(void.VoidB200Error):
        void.void_spmm(w.a.cpu(), w.b)
    small = void.VOIDTensor(torch.zeros(1, 16, 16, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"),
                            torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int64, device="cuda"),
                            (16, 16), (16, 16), 0, 1, 1.0)
    with pytest.raises(NotImplementedError):
        void.void_spmm(small, torch.zeros(16, 8, device="cuda"))
