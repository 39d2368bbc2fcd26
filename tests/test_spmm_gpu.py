"""GPU parity of the SpMM kernels through the Python operators (which call the C ABI):
int32 accumulators bit-exact, dequantised outputs within the path's tolerances
(INT8: rel 1e-3 after the fp16 cast; FP8: rel 1e-2), against reference-made fixtures and against
the CPU oracle on seeded inputs up to the benchmark sizes."""
import numpy as np
import pytest
import torch

import void_b200 as void
from void_b200 import workloads
from conftest import coo_to_csr, load_golden, rel_err
from oracle import void_oracle as vo

pytestmark = pytest.mark.gpu

INT8_TOL = 1e-3   # max|C - C_ref| / max|C_ref|, fp16 / bf16 outputs included
FP8_TOL = 1e-2


def _np(t):
    return t.detach().float().cpu().numpy()


def _int8_inputs(name):
    g = load_golden(name)
    a = void.csr_to_void(coo_to_csr(g), device="cuda")
    q = void.quantize_void_tensor(a)
    return g, q, torch.from_numpy(g["b_q"]).cuda(), torch.from_numpy(g["b_scales"]).cuda()


def test_int8_spmm_plumbing_workload_vs_reference():
    g, q, bq, bs = _int8_inputs("c1_plumbing.npz")
    acc = torch.zeros(512, 128, dtype=torch.int32, device="cuda")
    c = void.void_spmm_int8(q, bq, bs, acc_out=acc)
    void.check_device_status()
    assert c.dtype == torch.float32 and rel_err(_np(c), g["c_int8"]) < 1e-6
    ref_acc = vo.spmm_int8_acc(g["a_q"], _np(q.block_rows).astype(np.int32), _np(q.block_cols).astype(np.int32),
                               (512, 512), g["b_q"])
    assert np.array_equal(acc.cpu().numpy(), ref_acc)
    c16 = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16)
    assert c16.dtype == torch.float16 and rel_err(_np(c16), g["c_int8"]) < INT8_TOL
    assert np.array_equal(_np(c16), g["c_int8"].astype(np.float16).astype(np.float32))


def test_int8_spmm_small_cases_vs_reference():
    g, q, bq, bs = _int8_inputs("int8_small.npz")
    c_unit = void.void_spmm_int8(q, bq)                       # b_scale None -> 1.0
    assert np.array_equal(_np(c_unit), g["c_unit"])           # ragged M/K/N, empty tile rows
    c_scalar = void.void_spmm_int8(q, bq, float(g["b_scalar"][0]))
    assert rel_err(_np(c_scalar), g["c_scalar"]) < 1e-6
    c_float = void.void_spmm_int8(q, torch.from_numpy(g["b"]).cuda())   # fp32 B: quantised per tensor
    assert rel_err(_np(c_float), g["c_float_b"]) < 1e-6
    out = torch.full((200, 80), 7.0, device="cuda")
    assert void.void_spmm_int8(q, bq, out=out) is out and np.array_equal(_np(out), g["c_unit"])
    void.check_device_status()


def test_int8_exact_scales_is_true_per_block_dequant():
    g, q, bq, bs = _int8_inputs("int8_small.npz")
    c = void.void_spmm_int8(q, bq, bs, exact_scales=True)
    a_deq = np.zeros((224, 288), np.float32)
    for i in range(q.n_blocks):
        r, cc = int(g["block_rows"][i]), int(g["block_cols"][i])
        a_deq[r * 32:(r + 1) * 32, cc * 32:(cc + 1) * 32] = g["a_q"][i].astype(np.float32) * g["a_scales"][i]
    ref = a_deq[:200, :270].astype(np.float64) @ (g["b_q"].astype(np.float64) * g["b_scales"][None, :])
    assert rel_err(_np(c), ref) < 1e-5


def test_int8_spmm_empty_and_degenerate():
    import scipy.sparse as sp
    empty = void.quantize_void_tensor(void.csr_to_void(sp.csr_matrix((100, 70), dtype=np.float32), device="cuda"))
    b = torch.randint(-128, 128, (70, 48), dtype=torch.int8, device="cuda")
    c = void.void_spmm_int8(empty, b)
    assert c.shape == (100, 48) and not c.any()
    one = sp.lil_matrix((333, 555), dtype=np.float32)
    one[332, 554] = 2.5
    one[0, 0] = -1.0
    t = void.quantize_void_tensor(void.csr_to_void(one.tocsr(), device="cuda"))
    b = torch.randint(-128, 128, (555, 24), dtype=torch.int8, device="cuda")   # N not a multiple of 16
    c = void.void_spmm_int8(t, b)
    ref = vo.spmm_int8(_np(t.values).astype(np.int8), _np(t.scales), _np(t.block_rows).astype(np.int32),
                       _np(t.block_cols).astype(np.int32), (333, 555), _np(b).astype(np.int8))
    assert np.array_equal(_np(c), ref)
    void.check_device_status()


@pytest.mark.parametrize("shape,n", [((2048, 96), 64), ((96, 4096), 640), ((4096, 4096), 512)])
def test_int8_spmm_shapes_vs_oracle(shape, n):
    M, K = shape
    mask = workloads.uniform_mask(M // 32, K // 32, 0.9 if M == K else 0.5, seed=2)
    w = workloads.block_sparse(mask, n, seed=2)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    acc = torch.zeros(M, n, dtype=torch.int32, device="cuda")
    c = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16, acc_out=acc)
    void.check_device_status()
    args = (_np(q.values).astype(np.int8), _np(q.block_rows).astype(np.int32), _np(q.block_cols).astype(np.int32), (M, K))
    assert np.array_equal(acc.cpu().numpy(), vo.spmm_int8_acc(*args, bq.cpu().numpy()))
    ref = vo.spmm_int8(args[0], _np(q.scales), args[1], args[2], (M, K), bq.cpu().numpy(), col_scale=_np(bs))
    assert rel_err(_np(c), ref) < INT8_TOL
    assert np.array_equal(_np(c), ref.astype(np.float16).astype(np.float32))


def test_int8_spmm_launch_shapes_agree():
    """Panels per work item, ring depth and grid size change the schedule, never the result."""
    from void_b200 import _lib, _spmm
    w = workloads.headline(0.9)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    base = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16)
    for np_, stages, grid in [(1, 4, 37), (2, 5, 0), (4, 4, 148), (4, 5, 1000)]:
        out = torch.empty_like(base)
        _spmm.spmm(q.packed(), bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, panels_per_item=np_,
                   stages=stages, grid=grid)
        assert torch.equal(out, base), (np_, stages, grid)
    void.check_device_status()


def test_row_order_changes_the_schedule_only():
    """Launches without a plan take the tile rows by falling tile count (PackedTiles.row_order); the result has the
    bits of the launch that takes them in their own order, with one and several work items per CTA, and a list
    with entries outside the tensor is clamped instead of followed."""
    from void_b200 import _lib, _spmm
    for nbr, nbc, n, grid in ((37, 29, 384, 0), (37, 29, 384, 5), (128, 128, 512, 0), (3, 40, 100, 0)):
        mask = workloads.uniform_mask(nbr, nbc, 0.8, seed=nbr)
        mask[nbr // 2] = False
        w = workloads.block_sparse(mask, n, seed=nbr)
        q = void.quantize_void_tensor(w.a)
        bq, bs = void.quantize_cols_int8(w.b)
        p = q.packed()
        counts = (p.row_ptr[1:] - p.row_ptr[:-1]).cpu().numpy()
        order = p.row_order.cpu().numpy()
        assert sorted(order.tolist()) == list(range(nbr)) and np.all(np.diff(counts[order]) <= 0)
        outs = []
        for srt in (False, True):
            out = torch.full((nbr * 32, n), 7.0, dtype=torch.float16, device="cuda")
            _spmm.spmm(p, bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, grid=grid, sorted_rows=srt)
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), (nbr, nbc, n, grid)
    # a list that is not a permutation: nothing outside C is touched, the launch ends normally
    bad = p.row_order.clone()
    bad[0], bad[1] = -5, 10 ** 6
    keep, p.row_order = p.row_order, bad
    try:
        guard = torch.full((nbr * 32 + 64, n), 7.0, dtype=torch.float16, device="cuda")
        _spmm.spmm(p, bq, guard[32:32 + nbr * 32], scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs)
        torch.cuda.synchronize()
        assert bool((guard[:32] == 7.0).all()) and bool((guard[32 + nbr * 32:] == 7.0).all())
    finally:
        p.row_order = keep
    void.check_device_status()


@pytest.mark.parametrize("case", [(16, 16, 256, 0, torch.float16, 0), (9, 7, 200, 5, torch.bfloat16, 2),
                                  (5, 5, 128, 31, torch.float16, 1), (4, 4, 8, 0, torch.bfloat16, 3)])
def test_staged_tma_store_equals_direct_stores(case):
    """16-bit outputs through the shared-memory staging tile and a clipped TMA store: same bits as the direct stores,
    at ragged M and N, with biases and every activation, one and several work items per CTA."""
    from void_b200 import _lib, _spmm
    nbr, nbc, n, m_cut, dt, act = case
    mask = workloads.uniform_mask(nbr, nbc, 0.6, seed=n)
    mask[1] = False
    w = workloads.block_sparse(mask, n, seed=n)
    M = nbr * 32 - m_cut
    a = void.VOIDTensor(w.a.values, w.a.block_rows, w.a.block_cols, w.a.morton_codes, (M, nbc * 32), (32, 32), 0,
                        w.a.n_blocks, 0.0)
    q = void.quantize_void_tensor(a)
    bq, bs = void.quantize_cols_int8(w.b)
    gen = torch.Generator(device="cuda").manual_seed(1)
    bias, rb = torch.randn(n, device="cuda", generator=gen), torch.randn(M, device="cuda", generator=gen)
    outs = []
    for flags, grid, np_ in ((2, 0, 0), (0, 0, 0), (0, 3, 1), (0, 3, 2)):      # flags bit 1 = direct stores
        out = torch.full((M, n), 7.0, dtype=dt, device="cuda")
        _spmm.spmm(q.packed(), bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, bias=bias, row_bias=rb, act=act,
                   flags=flags, grid=grid, panels_per_item=np_)
        outs.append(out)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    void.check_device_status()


def test_linearity_and_row_permutation_properties():
    """Size-independent checks at the headline size: the int32 accumulators are linear in B, and a
    result row block depends only on its own tile row."""
    w = workloads.headline(0.9, seed=5)
    q = void.quantize_void_tensor(w.a)
    g = torch.Generator(device="cuda").manual_seed(0)
    b1 = torch.randint(-60, 60, (4096, 512), dtype=torch.int8, device="cuda", generator=g)
    b2 = torch.randint(-60, 60, (4096, 512), dtype=torch.int8, device="cuda", generator=g)
    accs = []
    for b in (b1, b2, b1 + b2):
        acc = torch.zeros(4096, 512, dtype=torch.int32, device="cuda")
        void.void_spmm_int8(q, b, acc_out=acc)
        accs.append(acc)
    assert torch.equal(accs[0] + accs[1], accs[2])
    dense = w.a.to_dense()
    assert dense.shape == (4096, 4096)


# How far each way of applying A's per-tile scales may be from the reference's output: 0 = every tile's fp32
# product scaled in registers (exact), 3 / 2 = scales folded into A as a sum of three / two E4M3 terms.
FP8_TERMS_TOL = {0: 1e-5, 3: 1e-4, 2: 2e-3}


@pytest.mark.parametrize("terms", [0, 3, 2])
def test_fp8_spmm_vs_reference_fixture(terms):
    g = load_golden("fp8_small.npz")
    a = void.csr_to_void(coo_to_csr(g), device="cuda")
    a8 = void.void_tensor_to_fp8(a)
    b8 = torch.from_numpy(g["b_fp8"]).cuda().view(torch.float8_e4m3fn)
    bs = torch.from_numpy(g["b_scale"]).cuda()
    tol = FP8_TERMS_TOL[terms]
    c = void.void_spmm_fp8(a8, b8, torch.float32, b_scale=bs, scale_terms=terms)
    assert rel_err(_np(c), g["c_block"]) < tol              # far inside the 1e-2 bar
    c16 = void.void_spmm_fp8(a8, b8, b_scale=bs, scale_terms=terms)      # default output dtype: fp16
    assert c16.dtype == torch.float16 and rel_err(_np(c16), g["c_f16"]) < FP8_TOL
    c_raw = void.void_spmm_fp8(a8, b8, torch.float32, scale_terms=terms)       # unit B scales
    assert rel_err(_np(c_raw), g["c_block_rawb"]) < tol
    # a floating-point B is used as it is, like the reference kernel does (the floating-point kernel on the
    # dequantised tiles; fp32 operands multiply as TF32: the reference's own 1e-3 bar)
    b32 = torch.from_numpy(g["b"]).cuda()
    c_fb = void.void_spmm_fp8(a8, b32, torch.float32, scale_terms=terms)
    assert c_fb.dtype == torch.float32 and rel_err(_np(c_fb), g["c_floatb"]) < 1e-3
    c_fb16 = void.void_spmm_fp8(a8, b32.half())
    assert c_fb16.dtype == torch.float16 and rel_err(_np(c_fb16), g["c_floatb"]) < 2e-3
    # one scale for all tiles: nothing to fold, every form is exact
    at = void.void_tensor_to_fp8(a, scale_mode="per_tensor")
    ct = void.void_spmm_fp8(at, b8, torch.float32, b_scale=bs, scale_terms=terms)
    assert rel_err(_np(ct), g["c_tensor"]) < 1e-5
    void.check_device_status()


def test_fp8_default_scale_terms_follow_the_output_type():
    g = load_golden("fp8_small.npz")
    a8 = void.void_tensor_to_fp8(void.csr_to_void(coo_to_csr(g), device="cuda"))
    b8 = torch.from_numpy(g["b_fp8"]).cuda().view(torch.float8_e4m3fn)
    bs = torch.from_numpy(g["b_scale"]).cuda()
    for dtype, terms in ((torch.float16, 2), (torch.bfloat16, 2), (torch.float32, 3)):
        assert torch.equal(void.void_spmm_fp8(a8, b8, dtype, b_scale=bs),
                           void.void_spmm_fp8(a8, b8, dtype, b_scale=bs, scale_terms=terms))
    with pytest.raises(ValueError):
        void.void_spmm_fp8(a8, b8, b_scale=bs, scale_terms=4)


@pytest.mark.parametrize("terms", [0, 2, 3])
@pytest.mark.parametrize("sparsity", [0.70, 0.80, 0.90, 0.95, 0.98])
def test_fp8_spmm_sparsity_sweep_vs_oracle(sparsity, terms):
    w = workloads.headline(sparsity, seed=1)
    a8 = void.void_tensor_to_fp8(w.a)
    b8, bs, _ = void.quantize_cols_fp8(w.b)
    c = void.void_spmm_fp8(a8, b8, torch.float16, b_scale=bs, scale_terms=terms)
    void.check_device_status()
    b_deq = vo.fp8_bytes_to_float(b8.view(torch.uint8).cpu().numpy()) * _np(bs)[None, :]
    ref = vo.spmm_fp8(a8.values_fp8.view(torch.uint8).cpu().numpy(), _np(a8.scaling_info.scale),
                      _np(a8.block_rows).astype(np.int32), _np(a8.block_cols).astype(np.int32), (4096, 4096), b_deq)
    assert rel_err(_np(c), ref) < FP8_TOL
    assert rel_err(_np(c), ref) < 2e-3                      # fp16 rounding (and, for two terms, 8-bit folded scales)
    # reference's own accuracy bar for FP8 SpMM: mean relative error < 0.3 against fp32 (tests/test_fp8.py:233-238)
    dense = (w.a.to_dense() @ w.b)
    mean_rel = ((c.float() - dense).abs().mean() / dense.abs().mean()).item()
    assert mean_rel < 0.3
