"""GPU parity of the format / index / quantisation kernels: bit-exact against the fixtures the
reference produced and against the CPU oracle on larger seeded inputs."""
import numpy as np
import pytest
import torch

import void_b200 as void
from conftest import coo_to_csr, load_golden
from oracle import void_oracle as vo

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["format_small.npz", "c1_plumbing.npz"])
def test_csr_to_void_and_tile_index(name):
    g = load_golden(name)
    a = void.csr_to_void(coo_to_csr(g), tile_size=32, device="cuda")
    assert a.n_blocks == int(g["meta"][0]) and a.nnz_original == int(g["meta"][1])
    assert a.density == float(g["density"][0])
    assert np.array_equal(a.block_rows.cpu().numpy(), g["block_rows"]) and a.block_rows.dtype == torch.int32
    assert np.array_equal(a.block_cols.cpu().numpy(), g["block_cols"])
    assert np.array_equal(a.morton_codes.cpu().numpy(), g["morton_codes"]) and a.morton_codes.dtype == torch.int64
    if "values" in g:
        assert np.array_equal(a.values.cpu().numpy(), g["values"])
    row_ptr, block_indices = a.get_row_block_info()
    assert row_ptr.dtype == torch.int32 and block_indices.dtype == torch.int32
    assert np.array_equal(row_ptr.cpu().numpy(), g["row_ptr"])
    assert np.array_equal(block_indices.cpu().numpy(), g["block_indices"])
    assert a.get_row_block_info()[0] is row_ptr  # cached


def test_csr_to_void_device_builder_equals_host_builder():
    import scipy.sparse as sp
    rs = np.random.RandomState(3)
    m = sp.random(1500, 2100, density=0.002, format="csr", dtype=np.float32, random_state=rs)
    m.data[::7] = 0.0                                           # stored zeros still activate their tiles
    dev = void.csr_to_void(m, tile_size=32, device="cuda")     # built by the CUDA library
    host = void.csr_to_void(m, tile_size=32, device="cpu")     # numpy restatement of the reference's loop
    f = vo.csr_to_void_fields(m)
    assert dev.n_blocks == host.n_blocks == f["n_blocks"] and dev.nnz_original == m.nnz and dev.density == host.density
    for k in ("values", "block_rows", "block_cols", "morton_codes"):
        assert torch.equal(getattr(dev, k).cpu(), getattr(host, k)), k
        assert np.array_equal(getattr(dev, k).cpu().numpy(), f[k]), k
    assert void.csr_to_void(m, device="cuda", dtype=torch.float16).values.dtype == torch.float16


def test_dense_to_void_vs_reference_output():
    g = load_golden("dense_small.npz")
    a = torch.from_numpy(g["matrix"]).cuda()
    for tag in ("t0", "t10"):
        v = void.dense_to_void(a, tile_size=32, threshold=float(g[tag + "_threshold"][0]))
        assert v.n_blocks == int(g[tag + "_meta"][0]) and v.nnz_original == int(g[tag + "_meta"][1])
        assert v.density == float(g[tag + "_density"][0]) and v.shape == (150, 210) and v.dtype == torch.float32
        for k in ("values", "block_rows", "block_cols", "morton_codes"):
            got = getattr(v, k).cpu().numpy()
            assert np.array_equal(got, g[tag + "_" + k]) and got.dtype == g[tag + "_" + k].dtype, (tag, k)
    e = void.dense_to_void(torch.zeros(40, 50, device="cuda"))
    assert [e.n_blocks, e.nnz_original] == g["empty_meta"].tolist() and e.density == 0.0 and e.values.shape == (0, 32, 32)
    assert torch.equal(void.dense_to_void(a).to_dense(), a)                          # round trip
    with pytest.raises(void.VoidB200Error):
        void.dense_to_void(a.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_dense_to_void_large_and_strided(dtype):
    gen = torch.Generator().manual_seed(4)
    keep = (torch.rand(70, 90, generator=gen) < 0.15).repeat_interleave(32, 0).repeat_interleave(32, 1)
    full = (torch.randn(70 * 32, 90 * 32, generator=gen) * keep)[:2231, :2870].to(dtype)
    wide = torch.zeros(2231, 3000, dtype=dtype)
    wide[:, :2870] = full
    v = void.dense_to_void(wide.cuda()[:, :2870])                                    # row pitch larger than N
    f = vo.dense_to_void_fields(full.float().numpy())
    assert v.n_blocks == f["n_blocks"] and v.nnz_original == f["nnz_original"] and v.dtype == dtype
    assert np.array_equal(v.block_rows.cpu().numpy(), f["block_rows"])
    assert np.array_equal(v.block_cols.cpu().numpy(), f["block_cols"])
    assert np.array_equal(v.morton_codes.cpu().numpy(), f["morton_codes"])
    assert np.array_equal(v.values.float().cpu().numpy(), f["values"])
    b = torch.randn(2870, 64, generator=gen).to(dtype).cuda()
    ref = full.float().cuda() @ b.float()
    assert (void.void_spmm(v, b).float() - ref).abs().max() <= 4e-3 * ref.abs().max()   # TF32 / 16-bit output rounding


def test_tile_index_large_random_grid():
    rng = np.random.default_rng(3)
    mask = rng.random((517, 1033)) > 0.93
    mask[100] = False
    mask[200] = True
    rows, cols = np.nonzero(mask)
    p = rng.permutation(len(rows))
    rows, cols = rows[p].astype(np.int32), cols[p].astype(np.int32)
    from void_b200.format import build_tile_index
    row_ptr, bidx = build_tile_index(torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda(), 517, 1033)
    ref_rp, ref_bi = vo.row_block_info(rows, cols, 517, 1033)
    assert np.array_equal(row_ptr.cpu().numpy(), ref_rp) and np.array_equal(bidx.cpu().numpy(), ref_bi)


def test_empty_and_single_block_tensors():
    import scipy.sparse as sp
    empty = void.csr_to_void(sp.csr_matrix((100, 70), dtype=np.float32), device="cuda")
    assert empty.n_blocks == 0 and empty.values.shape == (0, 32, 32)
    rp, bi = empty.get_row_block_info()
    assert rp.cpu().tolist() == [0] * 5 and bi.numel() == 0
    one = sp.lil_matrix((333, 555), dtype=np.float32)
    one[332, 554] = 2.5
    t = void.csr_to_void(one.tocsr(), device="cuda")
    assert t.n_blocks == 1 and t.padded_shape == (352, 576) and t.block_grid == (11, 18)
    assert t.block_rows.item() == 10 and t.block_cols.item() == 17 and t.values[0, 12, 10].item() == 2.5
    rp, bi = t.get_row_block_info()
    assert rp.cpu().tolist() == [0] * 11 + [1] and bi.cpu().tolist() == [0]
    assert torch.equal(t.to_dense().cpu(), torch.from_numpy(one.toarray()))


def test_int8_quantisation_matches_reference_bits():
    for name in ("c1_plumbing.npz", "int8_small.npz"):
        g = load_golden(name)
        a = void.csr_to_void(coo_to_csr(g), device="cuda")
        q = void.quantize_void_tensor(a)
        assert np.array_equal(q.values.cpu().numpy(), g["a_q"]) and q.values.dtype == torch.int8
        assert np.array_equal(q.scales.cpu().numpy(), g["a_scales"]) and not q.zero_points.any()
        bq, bs = void.quantize_cols_int8(torch.from_numpy(g["b"]).cuda())
        assert np.array_equal(bq.cpu().numpy(), g["b_q"]) and np.array_equal(bs.cpu().numpy(), g["b_scales"])
        # the reference's own route to per-column scales: quantize_tensor on the transpose
        qt, params = void.quantize_tensor(torch.from_numpy(g["b"]).cuda().t().contiguous(),
                                          void.IntQuantConfig(scale_mode=void.ScaleMode.PER_CHANNEL))
        assert np.array_equal(qt.t().cpu().numpy(), g["b_q"])
        assert np.array_equal(params.scale.reshape(-1).cpu().numpy(), g["b_scales"])


def test_int8_quantisation_edge_values():
    v = torch.zeros(3, 32, 32)
    v[0, 0, 0], v[0, 1, 1], v[0, 2, 2] = 2.0, -1.0, 0.0234375   # 0.0234375/scale = 1.5 -> 2 (half to even)
    v[1] = 0.0                                                   # all-zero tile: scale clamps to 1e-8
    v[2] = torch.linspace(-3, 3, 1024).reshape(32, 32)
    t = void.VOIDTensor(v.cuda(), torch.zeros(3, dtype=torch.int32).cuda(), torch.arange(3, dtype=torch.int32).cuda(),
                        torch.zeros(3, dtype=torch.int64).cuda(), (32, 96), (32, 32), 0, 3, 1.0)
    q = void.quantize_void_tensor(t)
    rq, rs = vo.quantize_int8_tiles(v.numpy())
    assert np.array_equal(q.values.cpu().numpy(), rq) and np.array_equal(q.scales.cpu().numpy(), rs)
    assert q.values[0, 0, 0].item() == 127 and q.values[0, 2, 2].item() == 2 and q.scales[1].item() == np.float32(1e-8)


def test_int8_per_tensor_b_matches_oracle():
    g = load_golden("int8_small.npz")
    b = torch.from_numpy(g["b"]).cuda()
    q, params = void.quantize_tensor(b, void.IntQuantConfig(scale_mode=void.ScaleMode.PER_TENSOR))
    scale = np.float32(max(np.abs(g["b"]).max() / np.float32(128), 1e-8))
    assert params.scale.item() == scale
    ref = np.clip(np.rint(g["b"] / scale), -128, 127).astype(np.int8)
    assert np.array_equal(q.cpu().numpy(), ref)


def test_fp8_quantisation_matches_reference_bits():
    g = load_golden("fp8_small.npz")
    a = void.csr_to_void(coo_to_csr(g), device="cuda")
    a8 = void.void_tensor_to_fp8(a)                       # per_block, e4m3
    assert a8.values_fp8.dtype == torch.float8_e4m3fn
    assert np.array_equal(a8.values_fp8.view(torch.uint8).cpu().numpy(), g["a_fp8"])
    s = a8.scaling_info
    assert np.array_equal(s.scale.cpu().numpy(), g["a_scale"]) and np.array_equal(s.scale_inv.cpu().numpy(), g["a_scale_inv"])
    assert np.array_equal(s.amax.cpu().numpy(), g["a_amax"])
    assert np.array_equal(s.amax_history.cpu().numpy(), g["a_amax_history"])
    b8, bs, bsi = void.quantize_cols_fp8(torch.from_numpy(g["b"]).cuda())
    assert np.array_equal(b8.view(torch.uint8).cpu().numpy(), g["b_fp8"])
    assert np.array_equal(bs.cpu().numpy(), g["b_scale"]) and np.array_equal(bsi.cpu().numpy(), g["b_scale_inv"])
    at = void.void_tensor_to_fp8(a, scale_mode="per_tensor")
    assert np.array_equal(at.values_fp8.view(torch.uint8).cpu().numpy(), g["at_fp8"])
    assert at.scaling_info.scale.item() == g["at_scale"][0]


def test_fp8_quantisation_subnormals_and_amax_kat():
    # literal known answers of the reference, tests/test_fp8.py:133-150
    kat = torch.tensor([[[1.0, 2.0], [3.0, 4.0]], [[5.0, 6.0], [7.0, 8.0]]]).cuda()
    assert void.compute_amax(kat, "per_tensor").item() == 8.0
    assert void.compute_amax(kat, "per_block").cpu().tolist() == [4.0, 8.0]
    # values down to the smallest E4M3 subnormal (2^-9 after scaling) and ties
    v = torch.zeros(2, 32, 32)
    v[0, 0, 0] = 448.0
    v[0, 0, 1:9] = torch.tensor([2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 0.00292, 1.0625, 1.1875, -17.0, 447.9])
    v[1] = torch.randn(32, 32, generator=torch.Generator().manual_seed(1)) * 1e-3
    q, info = void.quantize_to_fp8(v.cuda(), void.FP8Config(scale_mode="per_block"))
    rq, rs, rsi, ramax = vo.quantize_fp8_tiles(v.numpy())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), rq)
    assert np.array_equal(info.scale.cpu().numpy(), rs) and np.array_equal(info.scale_inv.cpu().numpy(), rsi)


def test_quantisers_on_headline_size_match_oracle():
    from void_b200 import workloads
    w = workloads.headline(0.9)
    q = void.quantize_void_tensor(w.a)
    rq, rs = vo.quantize_int8_tiles(w.a.values.cpu().numpy())
    assert np.array_equal(q.values.cpu().numpy(), rq) and np.array_equal(q.scales.cpu().numpy(), rs)
    a8 = void.void_tensor_to_fp8(w.a)
    fq, fs, _, _ = vo.quantize_fp8_tiles(w.a.values.cpu().numpy())
    assert np.array_equal(a8.values_fp8.view(torch.uint8).cpu().numpy(), fq)
    assert np.array_equal(a8.scaling_info.scale.cpu().numpy(), fs)
    bq, bs = void.quantize_cols_int8(w.b)
    rbq, rbs = vo.quantize_int8_cols(w.b.cpu().numpy())
    assert np.array_equal(bq.cpu().numpy(), rbq) and np.array_equal(bs.cpu().numpy(), rbs)
    b8, b8s, _ = void.quantize_cols_fp8(w.b)
    rb8, rb8s, _ = vo.quantize_fp8_cols(w.b.cpu().numpy())
    assert np.array_equal(b8.view(torch.uint8).cpu().numpy(), rb8) and np.array_equal(b8s.cpu().numpy(), rb8s)
