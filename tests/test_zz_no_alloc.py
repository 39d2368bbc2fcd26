"""The allocation-free entry point, void_spmm_i8_static_scratch.

Who needs it: an embedder that cannot give the library scratch memory - for example a serving
process whose allocator took the whole GPU at start-up (cudaMalloc fails from then on), a loop
that must not allocate after warm-up, or a foreign-language binding that owns no device
allocator.  For those callers the split-row SpMM keeps the int32 accumulators of split rows in an
array built into the library instead of in caller memory.

The test drives the entry point straight through the C ABI, twice in a row on the same inputs,
and requires the result to be bit-identical to what the ordinary entry point (caller-provided
scratch) produces: the partial sums are integers, so there is no tolerance to grant.  The second
call checks that nothing left behind by the first one (accumulators, counters) leaks into the
result.  The file sorts last so that a run stopping at the first failure has already run
every other test.
"""
import ctypes

import pytest
import torch

import void_b200 as void
from void_b200 import _lib, stream_k, workloads

pytestmark = pytest.mark.gpu


def _args(packed, plan, b, col_scale, out):
    a = _lib.SpmmArgs()
    a.tiles, a.tile_cols, a.tile_scales = packed.tiles.data_ptr(), packed.tile_cols.data_ptr(), packed.tile_scales.data_ptr()
    a.row_ptr, a.row_scale = packed.row_ptr.data_ptr(), packed.row_scale.data_ptr()
    a.nbr, a.nbc, a.nnz = packed.nbr, packed.nbc, packed.nnz
    a.b, a.ldb, a.K, a.N = b.data_ptr(), b.stride(0), b.shape[0], b.shape[1]
    a.col_scale, a.b_scale, a.bias = col_scale.data_ptr(), 1.0, None
    a.out, a.ldc, a.M = out.data_ptr(), out.stride(0), out.shape[0]
    a.out_dtype, a.act, a.scale_mode = _lib.OUT_DTYPE_CODE[out.dtype], _lib.ACT_GELU, _lib.SCALE_ROW_MEAN
    a.segs, a.cta_seg_ptr, a.n_cta = plan.segs.data_ptr(), plan.cta_seg_ptr.data_ptr(), plan.n_cta
    a.partials, a.counters = None, None          # the point of the entry point: no caller scratch
    a.status = _lib.status_word(out.device).data_ptr()
    a.panels_per_item = plan.np
    return a


def test_static_scratch_matches_caller_scratch_twice():
    lib = _lib.load()
    mask = workloads.zipf_mask(128, 512, 1.5, 300, 14.0, seed=13)
    w = workloads.block_sparse(mask, 256, seed=13)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    bq = bq.contiguous()
    wl = void.compute_stream_k_workload(q)
    plan = stream_k.stream_k_plan(q, 256, wl, n_cta=96)
    assert plan.n_slots > 0 and plan.n_counters > 0          # some tile rows really are split

    expected = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, out_dtype=torch.bfloat16, activation=_lib.ACT_GELU,
                                       n_cta=96)
    torch.cuda.synchronize()
    outs = [torch.full_like(expected, float("nan")) for _ in range(2)]
    for call in range(2):
        out = outs[call]
        args = _args(q.packed(), plan, bq, bs, out)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        status = lib.void_spmm_i8_static_scratch(ctypes.byref(args), plan.n_counters, _lib.stream_ptr())
        assert status == 0, lib.void_strerror(status)
        torch.cuda.synchronize()
        if call == 1:     # the first call on a device may load the library's image (array included); later ones take nothing
            assert torch.cuda.mem_get_info()[0] == free_before
        void.check_device_status()
        assert torch.equal(out, expected), "call %d differs from the caller-scratch result" % call


def test_static_scratch_refuses_split_rows_beyond_what_it_cleared():
    """A plan with more split rows than the caller declared: the rows beyond are skipped and reported through
    the status word; nothing outside the part of the array the call cleared is touched."""
    lib = _lib.load()
    mask = workloads.zipf_mask(128, 512, 1.5, 300, 14.0, seed=13)
    w = workloads.block_sparse(mask, 256, seed=13)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    bq = bq.contiguous()
    wl = void.compute_stream_k_workload(q)
    plan = stream_k.stream_k_plan(q, 256, wl, n_cta=96)
    assert plan.n_counters >= 2
    out = torch.zeros(q.shape[0], 256, dtype=torch.bfloat16, device="cuda")
    args = _args(q.packed(), plan, bq, bs, out)
    assert lib.void_spmm_i8_static_scratch(ctypes.byref(args), plan.n_counters - 1, _lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    with pytest.raises(void.VoidB200Error, match="does not fit"):
        void.check_device_status()
    # and a correct call afterwards is unaffected
    expected = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, out_dtype=torch.bfloat16, activation=_lib.ACT_GELU, n_cta=96)
    assert lib.void_spmm_i8_static_scratch(ctypes.byref(args), plan.n_counters, _lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    void.check_device_status()
    assert torch.equal(out, expected)


def test_static_scratch_rejects_oversized_plans():
    lib = _lib.load()
    mask = workloads.uniform_mask(4, 8, 0.5, seed=2)
    w = workloads.block_sparse(mask, 128, seed=2)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    wl = void.compute_stream_k_workload(q)
    plan = stream_k.stream_k_plan(q, 128, wl, n_cta=4)
    out = torch.empty(128, 128, device="cuda")
    args = _args(q.packed(), plan, bq.contiguous(), bs, out)
    too_many_rows = (8 << 20) // (plan.np * 16384) + 1
    assert lib.void_spmm_i8_static_scratch(ctypes.byref(args), too_many_rows, _lib.stream_ptr()) == -8
    assert lib.void_spmm_i8_static_scratch(ctypes.byref(args), 4097, _lib.stream_ptr()) == -8
    assert b"maximum" in lib.void_strerror(-8)
    args.segs = None                                          # without a plan there is nothing to park
    assert lib.void_spmm_i8_static_scratch(ctypes.byref(args), 0, _lib.stream_ptr()) == -1
