"""Paths that only run when something is wrong, exercised without any fault, trap or unbounded wait: a bounded
device-side wait that is made to run out (a test hook keeps one ring stage from ever being filled, the wait
limit is set to a few milliseconds), and a work plan that points outside the scratch it was given.  In both the
kernel returns in an orderly way with a code in the status word, and the next launch is correct."""
import pytest
import torch

import void_b200 as void
from void_b200 import _lib, _spmm, stream_k, workloads

pytestmark = pytest.mark.gpu

DROP_FIRST_GROUP = 1 << 16


def _small():
    mask = workloads.zipf_mask(64, 256, 1.5, 200, 10.0, seed=7)
    w = workloads.block_sparse(mask, 256, seed=7)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    return q, bq.contiguous(), bs


def test_bounded_wait_runs_out_with_a_status_and_the_next_launch_is_clean():
    q, bq, bs = _small()
    want = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16)
    torch.cuda.synchronize()
    void.check_device_status()
    out = torch.zeros_like(want)
    # every CTA's first group of tiles is never delivered; the consumer's wait is limited to 5 ms
    _spmm.spmm(q.packed(), bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, test_hooks=DROP_FIRST_GROUP | 5)
    with pytest.raises(void.VoidB200Error, match="wait gave up"):
        void.check_device_status()
    void.check_device_status()                                   # the word was cleared
    again = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16)   # tensor memory was given back, nothing hangs
    void.check_device_status()
    assert torch.equal(again, want)


def test_a_launch_that_gave_up_leaves_no_partial_sums_behind():
    q, bq, bs = _small()
    wl = void.compute_stream_k_workload(q)
    want = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, out_dtype=torch.float16, n_cta=48)
    plan = stream_k.stream_k_plan(q, 256, wl, n_cta=48)
    assert plan.n_counters > 0
    void.check_device_status()
    out = torch.zeros_like(want)
    _spmm.spmm(q.packed(), bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, plan=plan, test_hooks=DROP_FIRST_GROUP | 5)
    torch.cuda.synchronize()
    dirty = bool(plan.partials.any()) or bool(plan.counters.any())
    with pytest.raises(void.VoidB200Error):
        void.check_device_status()
    assert not plan.partials.any() and not plan.counters.any()   # cleared together with the status word
    again = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, out_dtype=torch.float16, n_cta=48)
    void.check_device_status()
    assert torch.equal(again, want), "dirty scratch before the reset: %s" % dirty


def test_plan_that_points_outside_its_scratch_is_reported_not_followed():
    q, bq, bs = _small()
    wl = void.compute_stream_k_workload(q)
    plan = stream_k.stream_k_plan(q, 256, wl, n_cta=48)
    assert plan.n_counters >= 2
    want = void.void_spmm_stream_k(q, bq, wl, b_scale=bs, out_dtype=torch.float16, n_cta=48)
    per_row = plan.np * 128 * 32
    guard = torch.zeros(plan.n_counters * per_row + 4096, dtype=torch.int32, device="cuda")
    short = _spmm.Plan(plan.segs, plan.cta_seg_ptr, plan.n_cta, plan.np, plan.n_chunks, plan.n_segs, plan.n_slots,
                       plan.n_counters, guard[:(plan.n_counters - 1) * per_row], torch.zeros_like(plan.counters),
                       plan.mode, plan.chunk_tiles)                # room for one split row less than the plan needs
    out = torch.zeros_like(want)
    _spmm.spmm(q.packed(), bq, out, scale_mode=_lib.SCALE_ROW_MEAN, col_scale=bs, plan=short)
    torch.cuda.synchronize()
    assert not guard[(plan.n_counters - 1) * per_row:].any()      # nothing was written behind the scratch
    with pytest.raises(void.VoidB200Error, match="does not fit"):
        void.check_device_status()
