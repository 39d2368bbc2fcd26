"""GPU parity of the fused GELU epilogue and of the Stream-K path: worker table bit-exact with the
reference's, per-worker int32 partial sums bit-exact and summing to the row accumulator, and the
load-balanced result identical to the plain kernel's."""
import numpy as np
import pytest
import torch

import void_b200 as void
from void_b200 import stream_k, workloads
from conftest import load_golden, rel_err
from oracle import void_oracle as vo

pytestmark = pytest.mark.gpu


def _np(t):
    return t.detach().float().cpu().numpy()


def _zipf_tensor(nbr=96, nbc=256, seed=7, n=192):
    mask = workloads.zipf_mask(nbr, nbc, 1.5, 200, 12.0, seed)
    mask[5] = False
    w = workloads.block_sparse(mask, n, seed)
    return w, void.quantize_void_tensor(w.a)


def test_activation_codes():
    # same table as the reference, tests/test_fusion.py:326-337
    assert [void.get_activation_code(x) for x in ("none", "relu", "gelu", "silu", "swish", "tanh", "sigmoid", "??")] == \
        [0, 1, 2, 3, 3, 4, 5, 0]
    assert void.get_activation_code(void.ActivationType.GELU) == 2


def test_gelu_epilogue_int8_vs_oracle():
    w, q = _zipf_tensor()
    bq, bs = void.quantize_cols_int8(w.b)
    bias = torch.randn(192, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    pre = void.void_spmm_int8(q, bq, bs)
    for b_ in (None, bias):
        ref = vo.gelu_tanh_sigmoid(_np(pre) + (0 if b_ is None else _np(b_)[None, :]))
        c32 = void.void_spmm_gelu(q, bq, b_, b_scale=bs)
        # exp / reciprocal in the kernel are the hardware approximations: a few 1e-7, bar is 1e-3
        assert c32.dtype == torch.float32 and rel_err(_np(c32), ref) < 1e-5
        c16 = void.void_spmm_gelu(q, bq, b_, b_scale=bs, out_dtype=torch.bfloat16)
        assert c16.dtype == torch.bfloat16
        # bf16 keeps 8 bits: within the 1e-3 bar before the cast, one bf16 ulp after it
        assert np.abs(_np(c16) - ref).max() <= 2.0 ** -8 * np.abs(ref).max()
    # matches torch's tanh GELU, which the reference kernel's sigmoid form equals to ~5e-7
    assert rel_err(_np(void.void_spmm_gelu(q, bq, b_scale=bs)),
                   _np(torch.nn.functional.gelu(pre, approximate="tanh"))) < 1e-5
    relu = void.void_spmm_relu(q, bq, b_scale=bs)
    assert torch.equal(relu, torch.relu(pre))
    void.check_device_status()


def test_gelu_epilogue_fp8():
    w, _ = _zipf_tensor(n=128)
    a8 = void.void_tensor_to_fp8(w.a)
    b8, bs, _ = void.quantize_cols_fp8(w.b)
    pre = void.void_spmm_fp8(a8, b8, torch.float32, b_scale=bs)
    c = void.void_spmm_gelu(a8, b8, b_scale=bs, output_dtype=torch.float32)
    assert rel_err(_np(c), vo.gelu_tanh_sigmoid(_np(pre))) < 1e-5


def test_gelu_on_floating_tensor_matches_torch_tanh_gelu():
    w, _ = _zipf_tensor()
    pre = void.void_spmm(w.a, w.b)
    assert rel_err(_np(void.void_spmm_gelu(w.a, w.b)), _np(torch.nn.functional.gelu(pre, approximate="tanh"))) < 1e-5
    with pytest.raises(TypeError):
        void.void_spmm_gelu(object(), w.b)


@pytest.mark.parametrize("tag", ["default", "w64", "w300_m4", "w7"])
def test_stream_k_table_bit_exact_with_reference(tag):
    g = load_golden("streamk_small.npz")
    nbr, nbc = (int(x) for x in g["grid"])
    n = len(g["block_rows"])
    t = void.VOIDTensor(torch.zeros(n, 32, 32, device="cuda"), torch.from_numpy(g["block_rows"]).cuda(),
                        torch.from_numpy(g["block_cols"]).cuda(), torch.zeros(n, dtype=torch.int64, device="cuda"),
                        (nbr * 32, nbc * 32), (32, 32), 0, n, n / (nbr * nbc))
    n_workers, total, req, max_work = (int(x) for x in g[tag + "_meta"])
    wl = void.compute_stream_k_workload(t, None if req < 0 else req, max_work)
    assert wl.n_workers == n_workers and wl.total_work == total
    assert wl.worker_rows.dtype == torch.int32 and wl.worker_needs_atomic.dtype == torch.bool
    assert np.array_equal(wl.worker_rows.cpu().numpy(), g[tag + "_rows"])
    assert np.array_equal(wl.worker_block_start.cpu().numpy(), g[tag + "_start"])
    assert np.array_equal(wl.worker_block_end.cpu().numpy(), g[tag + "_end"])
    assert np.array_equal(wl.worker_needs_atomic.cpu().numpy(), g[tag + "_atomic"])
    bal = void.analyze_workload_balance(t)
    got = [bal["n_rows"], bal["n_nonempty_rows"], bal["min_blocks_per_row"], bal["max_blocks_per_row"],
           bal["mean_blocks_per_row"], bal["std_blocks_per_row"], bal["imbalance_ratio"], bal["coefficient_of_variation"]]
    assert np.allclose(got, g["balance"], rtol=1e-6)


def test_stream_k_empty_tensor_raises_like_reference():
    t = void.VOIDTensor(torch.zeros(0, 32, 32, device="cuda"), torch.zeros(0, dtype=torch.int32, device="cuda"),
                        torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(0, dtype=torch.int64, device="cuda"),
                        (64, 64), (32, 32), 0, 0, 0.0)
    with pytest.raises(ZeroDivisionError):
        void.compute_stream_k_workload(t)


def test_stream_k_worker_partials_bit_exact():
    w, q = _zipf_tensor()
    bq, bs = void.quantize_cols_int8(w.b)
    wl = void.compute_stream_k_workload(q, n_workers=300, max_work_per_worker=4)
    assert wl.worker_needs_atomic.any() and not wl.worker_needs_atomic.all()
    plan = stream_k.stream_k_plan(q, 192, wl, per_worker=True, n_cta=24)
    segs = plan.segs.cpu().numpy().reshape(-1, 8)[:plan.n_segs]
    parts = torch.zeros(plan.n_segs, 32, 192, dtype=torch.int32, device="cuda")
    acc = torch.zeros(96 * 32, 192, dtype=torch.int32, device="cuda")
    c = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, worker_partials=parts, acc_out=acc, n_cta=24)
    void.check_device_status()
    args = (_np(q.values).astype(np.int8), _np(q.block_rows).astype(np.int32), _np(q.block_cols).astype(np.int32),
            q.shape)
    b_np = bq.cpu().numpy()
    ref_acc = vo.spmm_int8_acc(*args, b_np)
    assert np.array_equal(acc.cpu().numpy(), ref_acc)
    # one segment per worker of the table and per column chunk of the plan
    chunk_cols = plan.np * 128
    for ch in range(plan.n_chunks):
        worker_segs = segs[(segs[:, 3] > segs[:, 2]) & (segs[:, 1] == ch)]
        assert np.array_equal(worker_segs[:, 0], wl.worker_rows.cpu().numpy())
        assert np.array_equal(worker_segs[:, 2], wl.worker_block_start.cpu().numpy())
        assert np.array_equal(worker_segs[:, 3], wl.worker_block_end.cpu().numpy())
    parts_np = parts.cpu().numpy()
    total = np.zeros_like(ref_acc)
    rng = np.random.default_rng(0)
    check = set(rng.choice(len(segs), 40, replace=False).tolist())
    for i, (row, ch, t0, t1, nseg, slot0, idx, ctr) in enumerate(segs):
        total[row * 32:(row + 1) * 32] += parts_np[i]
        if i in check:
            cols = slice(ch * chunk_cols, min((ch + 1) * chunk_cols, 192))
            ref_part = vo.spmm_int8_acc(*args, b_np, t_range=(int(t0), int(t1)))[row * 32:(row + 1) * 32]
            assert np.array_equal(parts_np[i][:, cols], ref_part[:, cols])
            assert not np.delete(parts_np[i], np.arange(cols.start, cols.stop), axis=1).any()
    assert np.array_equal(total, ref_acc)                     # sum of partials = row accumulator
    plain = void.void_spmm_int8(q, bq, bs)
    assert torch.equal(c, plain)


@pytest.mark.parametrize("n_cta", [None, 5, 64, 500])
def test_stream_k_result_equals_plain_kernel(n_cta):
    w, q = _zipf_tensor(nbr=128, nbc=512, seed=11, n=256)
    bq, bs = void.quantize_cols_int8(w.b)
    plain = void.void_spmm_int8(q, bq, bs, out_dtype=torch.bfloat16, activation=2)
    for rep in range(3):                                       # counters must be left clean between calls
        c = void.void_spmm_stream_k(q, bq, b_scale=bs, out_dtype=torch.bfloat16, activation=2, n_cta=n_cta)
        assert torch.equal(c, plain)
    void.check_device_status()


def test_stream_k_power_law_benchmark_size():
    w = workloads.power_law()
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    wl = void.compute_stream_k_workload(q)
    rp = q.get_row_block_info()[0].cpu().numpy()
    rows, start, end, atomic = vo.stream_k_workload(rp, q.n_blocks)
    assert wl.n_workers == len(rows) and np.array_equal(wl.worker_block_start.cpu().numpy(), start)
    assert np.array_equal(wl.worker_needs_atomic.cpu().numpy(), atomic)
    acc = torch.zeros(16384, 256, dtype=torch.int32, device="cuda")
    c = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, out_dtype=torch.bfloat16, activation=2, acc_out=acc)
    void.check_device_status()
    args = (_np(q.values).astype(np.int8), _np(q.block_rows).astype(np.int32), _np(q.block_cols).astype(np.int32),
            q.shape)
    assert np.array_equal(acc.cpu().numpy(), vo.spmm_int8_acc(*args, bq.cpu().numpy()))
    ref = vo.gelu_tanh_sigmoid(vo.spmm_int8(args[0], _np(q.scales), args[1], args[2], q.shape, bq.cpu().numpy(),
                                            col_scale=_np(bs)))
    assert np.abs(_np(c) - ref).max() <= 2.0 ** -8 * np.abs(ref).max()
    assert torch.equal(c, void.void_spmm_int8(q, bq, bs, out_dtype=torch.bfloat16, activation=2))
    prof = void.analyze_workload(q)
    assert prof.use_stream_k and prof.imbalance_ratio > 5
