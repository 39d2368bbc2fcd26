"""Pins the CPU oracle to the reference: every oracle function is compared with fixtures that the
reference itself produced (tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import pytest

from conftest import coo_to_csr, load_golden, rel_err
from oracle import void_oracle as vo


def test_morton_known_values():
    # morton_encode(x, y) = spread(x) | spread(y) << 1, void/format.py:15-25
    assert vo.morton_encode_batch(np.array([0, 1, 0, 1, 2, 3]), np.array([0, 0, 1, 1, 0, 5])).tolist() == \
        [0, 1, 2, 3, 4, 0b100111]
    assert int(vo.morton_encode_batch(np.array([65535]), np.array([65535]))[0]) == 0xFFFFFFFF


@pytest.mark.parametrize("name", ["format_small.npz", "c1_plumbing.npz"])
def test_csr_to_void_fields(name):
    g = load_golden(name)
    f = vo.csr_to_void_fields(coo_to_csr(g))
    assert f["n_blocks"] == int(g["meta"][0]) and f["nnz_original"] == int(g["meta"][1])
    assert f["density"] == float(g["density"][0])
    for k in ("block_rows", "block_cols", "morton_codes"):
        assert np.array_equal(f[k], g[k]) and f[k].dtype == g[k].dtype, k
    if "values" in g:
        assert np.array_equal(f["values"], g["values"])
    M, K = f["shape"]
    row_ptr, bidx = vo.row_block_info(f["block_rows"], f["block_cols"], (M + 31) // 32, (K + 31) // 32)
    assert np.array_equal(row_ptr, g["row_ptr"]) and row_ptr.dtype == np.int32
    assert np.array_equal(bidx, g["block_indices"]) and bidx.dtype == np.int32


def test_dense_to_void_fields():
    g = load_golden("dense_small.npz")
    for tag in ("t0", "t10"):
        f = vo.dense_to_void_fields(g["matrix"], float(g[tag + "_threshold"][0]))
        assert f["n_blocks"] == int(g[tag + "_meta"][0]) and f["nnz_original"] == int(g[tag + "_meta"][1])
        assert f["density"] == float(g[tag + "_density"][0])
        for k in ("values", "block_rows", "block_cols", "morton_codes"):
            assert np.array_equal(f[k], g[tag + "_" + k]) and f[k].dtype == g[tag + "_" + k].dtype, (tag, k)
    assert int(g["t10_meta"][0]) < int(g["t0_meta"][0])            # the threshold drops the faint tiles
    e = vo.dense_to_void_fields(np.zeros((40, 50), np.float32))
    assert [e["n_blocks"], e["nnz_original"]] == g["empty_meta"].tolist() and e["density"] == 0.0


def test_c1_is_fully_dense_in_blocks():
    g = load_golden("c1_plumbing.npz")
    assert int(g["meta"][0]) == 256  # density 0.1 fills every 32x32 tile of the 16x16 block grid


def test_int8_quantisation_bit_exact():
    for name in ("c1_plumbing.npz", "int8_small.npz"):
        g = load_golden(name)
        f = vo.csr_to_void_fields(coo_to_csr(g))
        q, s = vo.quantize_int8_tiles(f["values"])
        assert np.array_equal(q, g["a_q"]) and np.array_equal(s, g["a_scales"])
        bq, bs = vo.quantize_int8_cols(g["b"])
        assert np.array_equal(bq, g["b_q"]) and np.array_equal(bs, g["b_scales"])


def test_int8_scale_uses_128():
    # absmax / 128, not / 127: void/int_quant.py:204
    v = np.zeros((1, 32, 32), np.float32)
    v[0, 0, 0], v[0, 1, 1], v[0, 2, 2] = 2.0, -1.0, 0.0234375
    q, s = vo.quantize_int8_tiles(v)
    assert s[0] == np.float32(2.0 / 128) and q[0, 0, 0] == 127 and q[0, 1, 1] == -64
    assert q[0, 2, 2] == 2  # 1.5 rounds half to even


def test_int8_spmm_c1():
    g = load_golden("c1_plumbing.npz")
    f = vo.csr_to_void_fields(coo_to_csr(g))
    c = vo.spmm_int8(g["a_q"], g["a_scales"], f["block_rows"], f["block_cols"], f["shape"], g["b_q"],
                     col_scale=g["b_scales"])
    assert rel_err(c, g["c_int8"]) < 1e-6
    # mean-scale semantic differs visibly from per-block dequantisation on this input
    a = coo_to_csr(g).toarray()
    assert rel_err(c, a @ g["b"]) > 1e-3


def test_fp_spmm_c1_and_small():
    # the reference's fp32 void_spmm (void/ops.py:148-217) run through the Triton interpreter
    g = load_golden("c1_plumbing.npz")
    f = vo.csr_to_void_fields(coo_to_csr(g))
    c = vo.spmm_fp(f["values"], f["block_rows"], f["block_cols"], f["shape"], g["b"])
    assert rel_err(c, g["c_fp32"]) < 1e-6
    assert rel_err(c, coo_to_csr(g).toarray() @ g["b"]) < 1e-5
    g = load_golden("fp_small.npz")
    f = vo.csr_to_void_fields(coo_to_csr(g))
    assert np.array_equal(f["block_rows"], g["block_rows"]) and np.array_equal(f["block_cols"], g["block_cols"])
    args = (f["values"], f["block_rows"], f["block_cols"], f["shape"])
    c = vo.spmm_fp(*args, g["b"])
    assert c.shape == (200, 80) and rel_err(c, g["c_fp32"]) < 1e-6
    assert not c[32:64].any() and not c[128:160].any()                    # empty tile rows stay zero
    assert rel_err(vo.spmm_fp(*args, g["x"][:, None])[:, 0], g["y_spmv"]) < 1e-6
    assert rel_err(vo.gelu_tanh_sigmoid(c), g["gelu"]) < 1e-6
    assert rel_err(vo.gelu_tanh_sigmoid(c + g["bias"][None, :]), g["gelu_bias"]) < 1e-6
    # bias per output row (the linear-layer kernel, void/fusion.py:201-304) and the two-layer MLP built on it
    assert rel_err(vo.gelu_tanh_sigmoid(c + g["bias1"][:, None]), g["rowbias_gelu"]) < 1e-6
    assert rel_err(vo.silu(c + g["bias1"][:, None]), g["rowbias_silu"]) < 1e-6
    import scipy.sparse as sp
    f2 = vo.csr_to_void_fields(sp.csr_matrix((g["w2_data"], (g["w2_row"], g["w2_col"])), shape=(70, 200)))
    w2 = (f2["values"], f2["block_rows"], f2["block_cols"], f2["shape"])
    assert rel_err(vo.sparse_mlp(args, w2, g["b"].T, g["bias1"], g["bias2"]), g["mlp"]) < 1e-6
    # fp16 tiles and fp16 B: products in fp32, result rounded to fp16 once
    c16 = vo.spmm_fp(f["values"].astype(np.float16), *args[1:], g["b"].astype(np.float16))
    assert rel_err(c16.astype(np.float16).astype(np.float32), g["c_f16"]) < 1e-3
    # Stream-K: the sum of the workers' partial products is the plain product (void/stream_k.py:198-219)
    rp, _ = vo.row_block_info(f["block_rows"], f["block_cols"], 7, 9)
    rows, start, end, atomic = vo.stream_k_workload(rp, len(f["block_rows"]), 12, 2)
    assert len(rows) == int(g["stream_k_meta"][0]) and atomic.any()
    total = np.zeros_like(c)
    for r, t0, t1 in zip(rows, start, end):
        total[r * 32:(r + 1) * 32] += vo.spmm_fp(*args, g["b"], t_range=(int(t0), int(t1)))[r * 32:(r + 1) * 32]
    assert rel_err(total, g["stream_k"]) < 1e-6 and rel_err(g["stream_k"], g["c_fp32"]) < 1e-6


def test_backward_matches_reference_autograd():
    g = load_golden("backward_small.npz")
    f = vo.csr_to_void_fields(coo_to_csr(g))
    assert rel_err(vo.spmm_fp(f["values"], f["block_rows"], f["block_cols"], f["shape"], g["b"]), g["c"]) < 1e-6
    gv, gb = vo.spmm_backward(f["values"], f["block_rows"], f["block_cols"], f["shape"], g["b"], g["grad_c"])
    assert gv.shape == g["grad_values"].shape and rel_err(gv, g["grad_values"]) < 1e-6
    assert gb.shape == (150, 72) and rel_err(gb, g["grad_b"]) < 1e-6
    # against dense calculus: dB = A^T dC, and dA restricted to the stored tiles
    a = coo_to_csr(g).toarray()
    assert rel_err(gb, a.T @ g["grad_c"]) < 1e-5
    full = np.zeros((192, 160), np.float32)
    full[:180, :150] = g["grad_c"] @ g["b"].T
    for i, (r, c) in enumerate(zip(f["block_rows"], f["block_cols"])):
        assert np.allclose(gv[i], full[r * 32:(r + 1) * 32, c * 32:(c + 1) * 32], rtol=1e-4, atol=1e-4)


def test_int8_spmm_small_cases():
    g = load_golden("int8_small.npz")
    shape = tuple(int(x) for x in g["shape"])
    args = (g["a_q"], g["a_scales"], g["block_rows"], g["block_cols"], shape, g["b_q"])
    assert rel_err(vo.spmm_int8(*args), g["c_unit"]) < 1e-6
    assert np.array_equal(vo.spmm_int8(*args), g["c_unit"])
    assert rel_err(vo.spmm_int8(*args, b_scale=float(g["b_scalar"][0])), g["c_scalar"]) < 1e-6
    # empty tile rows give exact zeros
    row_ptr, _ = vo.row_block_info(g["block_rows"], g["block_cols"], 7, 9)
    for r in np.nonzero(np.diff(row_ptr) == 0)[0]:
        assert not g["c_unit"][r * 32:(r + 1) * 32].any()
    # accumulators are what the kernel multiplies by the mean scale
    acc = vo.spmm_int8_acc(g["a_q"], g["block_rows"], g["block_cols"], shape, g["b_q"])
    rs = vo.int8_row_scale(g["a_scales"], g["block_rows"], g["block_cols"], shape)
    assert np.array_equal((acc.astype(np.float32) * np.repeat(rs, 32)[:, None])[:shape[0]], g["c_unit"])


def test_c_restatement_equals_numpy_oracle_and_reference():
    if vo.c_library() is None:
        pytest.skip("no C compiler")
    g = load_golden("int8_small.npz")                                   # ragged M / K / N, empty tile rows
    shape = tuple(int(x) for x in g["shape"])
    args = (g["a_q"], g["a_scales"], g["block_rows"], g["block_cols"], shape, g["b_q"])
    out, acc = vo.spmm_int8_c(*args, want_acc=True)
    assert np.array_equal(acc, vo.spmm_int8_acc(g["a_q"], g["block_rows"], g["block_cols"], shape, g["b_q"]))
    assert np.array_equal(out, vo.spmm_int8(*args)) and rel_err(out, g["c_unit"]) < 1e-6
    assert rel_err(vo.spmm_int8_c(*args, b_scale=float(g["b_scalar"][0])), g["c_scalar"]) < 1e-6
    g = load_golden("c1_plumbing.npz")
    f = vo.csr_to_void_fields(coo_to_csr(g))
    c = vo.spmm_int8_c(g["a_q"], g["a_scales"], f["block_rows"], f["block_cols"], f["shape"], g["b_q"],
                       col_scale=g["b_scales"])
    assert rel_err(c, g["c_int8"]) < 1e-6


def test_fp8_amax_known_answers():
    # the literal known-answer test of the reference, tests/test_fp8.py:133-150
    g = load_golden("fp8_small.npz")
    assert g["kat_amax_tensor"].tolist() == [8.0] and g["kat_amax_block"].tolist() == [4.0, 8.0]
    kat = np.array([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], np.float32)
    _, _, _, amax = vo.quantize_fp8_tiles(kat)
    assert amax.tolist() == [4.0, 8.0]


def test_fp8_quantisation_bit_exact():
    g = load_golden("fp8_small.npz")
    f = vo.csr_to_void_fields(coo_to_csr(g))
    q, s, si, amax = vo.quantize_fp8_tiles(f["values"])
    assert np.array_equal(q, g["a_fp8"]) and np.array_equal(s, g["a_scale"])
    assert np.array_equal(si, g["a_scale_inv"]) and np.array_equal(amax, g["a_amax"])
    assert np.array_equal(g["a_amax_history"][:, 0], amax) and not g["a_amax_history"][:, 1:].any()
    bq, bs, bsi = vo.quantize_fp8_cols(g["b"])
    assert np.array_equal(bq, g["b_fp8"]) and np.array_equal(bs, g["b_scale"]) and np.array_equal(bsi, g["b_scale_inv"])


def test_fp8_spmm():
    g = load_golden("fp8_small.npz")
    shape = tuple(int(x) for x in g["shape"])
    b_deq = vo.fp8_bytes_to_float(g["b_fp8"]) * g["b_scale"][None, :]
    c = vo.spmm_fp8(g["a_fp8"], g["a_scale"], g["block_rows"], g["block_cols"], shape, b_deq)
    assert rel_err(c, g["c_block"]) < 1e-6
    # B scales factor out of the sum: raw-B result times the column scales
    c_raw = vo.spmm_fp8(g["a_fp8"], g["a_scale"], g["block_rows"], g["block_cols"], shape,
                        vo.fp8_bytes_to_float(g["b_fp8"]))
    assert rel_err(c_raw, g["c_block_rawb"]) < 1e-6
    assert rel_err(c_raw * g["b_scale"][None, :], g["c_block"]) < 1e-6
    ct = vo.spmm_fp8(g["at_fp8"], g["at_scale"], g["block_rows"], g["block_cols"], shape, b_deq, per_tensor=True)
    assert rel_err(ct, g["c_tensor"]) < 1e-6
    assert rel_err(c.astype(np.float16).astype(np.float32), g["c_f16"]) < 1e-3
    # a floating-point B is used as it is
    cf = vo.spmm_fp8(g["a_fp8"], g["a_scale"], g["block_rows"], g["block_cols"], shape, g["b"])
    assert rel_err(cf, g["c_floatb"]) < 1e-6


def test_gelu_matches_reference_kernel():
    g = load_golden("gelu_small.npz")
    assert rel_err(vo.gelu_tanh_sigmoid(g["pre"]), g["post"]) < 1e-6
    assert rel_err(vo.gelu_tanh_sigmoid(g["pre"] + g["bias"][None, :]), g["post_bias"]) < 1e-6


@pytest.mark.parametrize("tag", ["default", "w64", "w300_m4", "w7"])
def test_stream_k_table(tag):
    g = load_golden("streamk_small.npz")
    nbr, nbc = (int(x) for x in g["grid"])
    row_ptr, _ = vo.row_block_info(g["block_rows"], g["block_cols"], nbr, nbc)
    n_workers, total, req, max_work = (int(x) for x in g[tag + "_meta"])
    rows, start, end, atomic = vo.stream_k_workload(row_ptr, total, None if req < 0 else req, max_work)
    assert len(rows) == n_workers
    assert np.array_equal(rows, g[tag + "_rows"]) and np.array_equal(start, g[tag + "_start"])
    assert np.array_equal(end, g[tag + "_end"]) and np.array_equal(atomic, g[tag + "_atomic"])
    assert int((end - start).sum()) == total  # total_work == n_blocks, tests/test_advanced_features.py:705-735


def test_workload_balance():
    g = load_golden("streamk_small.npz")
    nbr, nbc = (int(x) for x in g["grid"])
    row_ptr, _ = vo.row_block_info(g["block_rows"], g["block_cols"], nbr, nbc)
    b = vo.workload_balance(row_ptr)
    got = [b["n_rows"], b["n_nonempty_rows"], b["min_blocks_per_row"], b["max_blocks_per_row"],
           b["mean_blocks_per_row"], b["std_blocks_per_row"], b["imbalance_ratio"], b["coefficient_of_variation"]]
    assert np.allclose(got, g["balance"], rtol=1e-6)


def test_shard_rows_cover_and_rebase():
    g = load_golden("streamk_small.npz")
    nbr = int(g["grid"][0])
    for world in (1, 2, 3, 4, 8):
        seen = []
        for rank in range(world):
            start, end, idx, local_rows = vo.shard_rows(g["block_rows"], nbr, world, rank)
            assert start == rank * ((nbr + world - 1) // world)
            assert (np.diff(idx) > 0).all()  # original order kept
            assert np.array_equal(local_rows, g["block_rows"][idx] - start)
            assert ((local_rows >= 0) & (local_rows < max(end - start, 1))).all()
            seen.append(idx)
        assert np.array_equal(np.sort(np.concatenate(seen)), np.arange(len(g["block_rows"])))


def test_sharding_matches_reference_output():
    """Ranges, kept tiles (in kept order), rebased rows and local shape of all three strategies against the
    output of the reference's own shard_void_tensor (shard_small.npz), including a remainder and ranks past
    the end of the grid."""
    g = load_golden("shard_small.npz")
    shape = tuple(int(x) for x in g["shape"])
    for strategy in ("row_wise", "column_wise", "block_wise"):
        for world in (int(w) for w in g["worlds"]):
            for rank in range(world):
                tag = "%s_w%d_r%d_" % (strategy, world, rank)
                got = vo.shard(g["block_rows"], g["block_cols"], shape, world, rank, strategy)
                meta = [int(x) for x in g[tag + "meta"]]
                assert np.array_equal(got["ids"], g[tag + "ids"]), tag
                assert np.array_equal(got["rows"], g[tag + "rows"]), tag
                assert np.array_equal(got["cols"], g[tag + "cols"]), tag
                assert list(got["row_range"]) + list(got["col_range"]) + list(got["shape"]) == meta[:6], tag
                assert len(got["ids"]) == meta[6] and tuple(meta[7:9]) == shape
