"""Sharded SpMM on one GPU: every rank's shard is computed in turn and the concatenation of the
row shards must equal the unsharded result bit for bit (same kernel, independent tile rows)."""
import numpy as np
import pytest
import torch

import void_b200 as void
from void_b200 import workloads
from oracle import void_oracle as vo

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_row_shards_concatenate_to_unsharded(world):
    mask = workloads.uniform_mask(70, 40, 0.8, seed=4)
    w = workloads.block_sparse(mask, 160, seed=4)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    full_acc = torch.zeros(70 * 32, 160, dtype=torch.int32, device="cuda")
    full = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16, acc_out=full_acc)
    outs = []
    for rank in range(world):
        d = void.shard_void_tensor(q, void.ShardingStrategy.ROW_WISE, world_size=world, rank=rank)
        start, end, idx, local_rows = vo.shard_rows(q.block_rows.cpu().numpy(), 70, world, rank)
        assert d.local_row_range == (start, end) and d.local_col_range == (0, 40)
        assert np.array_equal(d.local_tensor.block_rows.cpu().numpy(), local_rows)
        assert torch.equal(d.local_tensor.values, q.values[torch.from_numpy(idx).cuda()])   # original order kept
        assert d.local_tensor.shape == ((end - start) * 32, 40 * 32) and d.global_shape == q.shape
        outs.append(void.distributed_void_spmm(d, bq, b_scale=bs, out_dtype=torch.float16, gather_output=False))
    cat = torch.cat(outs)[:70 * 32]
    assert torch.equal(cat, full)
    void.check_device_status()
    # and against the oracle on the same input, not only against the unsharded CUDA result: every rank's shard is
    # the oracle's product of the oracle's shard (int32 accumulators bit for bit, fp16 output within 1e-3)
    qv, qs = q.values.cpu().numpy(), q.scales.cpu().numpy()
    rows_np, cols_np = q.block_rows.cpu().numpy(), q.block_cols.cpu().numpy()
    bq_np, bs_np = bq.cpu().numpy(), bs.cpu().numpy()
    assert np.array_equal(full_acc.cpu().numpy(), vo.spmm_int8_acc(qv, rows_np, cols_np, q.shape, bq_np))
    for rank in range(world):
        sh = vo.shard(rows_np, cols_np, q.shape, world, rank, "row_wise")
        if len(sh["ids"]) == 0:
            assert not outs[rank].any()
            continue
        ref = vo.spmm_int8(qv[sh["ids"]], qs[sh["ids"]], sh["rows"], sh["cols"], sh["shape"], bq_np, col_scale=bs_np)
        got = outs[rank].float().cpu().numpy()[:ref.shape[0]]
        assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()


def test_product_by_column_panels_equals_whole_product():
    # the panel-wise first step (B arriving in column panels) on one rank: same bits as the one-launch product
    mask = workloads.uniform_mask(40, 24, 0.7, seed=6)
    w = workloads.block_sparse(mask, 416, seed=6)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    full = void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16)
    d = void.shard_void_tensor(q, world_size=1, rank=0)
    for cols in (128, 160, 416, 1000):
        got, b_back = void.broadcast_spmm_overlapped(d, bq, bs, panel_cols=cols, out_dtype=torch.float16)
        assert b_back is bq and torch.equal(got, full), cols
    void.check_device_status()


def test_fp8_and_float_tensors_shard_without_crashing():
    mask = workloads.uniform_mask(16, 16, 0.6, seed=9)
    w = workloads.block_sparse(mask, 64, seed=9)
    d = void.shard_void_tensor(w.a, world_size=4, rank=1)      # the reference raises TypeError here
    assert isinstance(d.local_tensor, void.VOIDTensor) and d.local_row_range == (4, 8)
    a8 = void.void_tensor_to_fp8(w.a)
    b8, bs, _ = void.quantize_cols_fp8(w.b)
    full = void.void_spmm_fp8(a8, b8, b_scale=bs)
    parts = [void.distributed_void_spmm(void.shard_void_tensor(a8, world_size=4, rank=r), b8, b_scale=bs,
                                        gather_output=False) for r in range(4)]
    assert torch.equal(torch.cat(parts), full)
    with pytest.raises(ValueError):
        void.shard_void_tensor(w.a, "diagonal", world_size=2, rank=0)


def test_sharded_generator_matches_global_mask():
    shard, (start, end), nnz = workloads.sharded_int8(M=4096, N=64, block_sparsity=0.9, seed=3, world_size=4, rank=2)
    mask = workloads.uniform_mask(128, 128, 0.9, 3)
    assert (start, end) == (64, 96) and nnz == int(mask.sum()) and shard.n_blocks == int(mask[64:96].sum())
    assert shard.shape == (32 * 32, 4096)
    rp, _ = shard.get_row_block_info()
    assert np.array_equal(np.diff(rp.cpu().numpy()), mask[64:96].sum(axis=1))


@pytest.mark.parametrize("mode", ["slots", "atomic"])
@pytest.mark.parametrize("strategy", [void.ShardingStrategy.COLUMN_WISE, void.ShardingStrategy.BLOCK_WISE])
@pytest.mark.parametrize("world", [2, 3])
def test_in_kernel_reduction_bookkeeping_on_one_gpu(strategy, world, mode):
    """The cross-rank reduction of the SpMM kernel with every "rank" played by this one GPU, one launch after the
    other.  "atomic": each launch adds its int32 partial tiles into the owner's accumulator and bumps the owner's
    counter, the last one finishes the row; accumulators and counters must be left at zero.  "slots": each launch
    stores its partial tiles into its own slot of the owner's scratch and the owner adds the slots afterwards.
    Either way the owners' rows together must be the unsharded product bit for bit, in any launch order."""
    from void_b200 import reduce as vr
    mask = workloads.uniform_mask(22, 19, 0.7, seed=12)
    mask[5] = False                                              # a tile row nobody holds a tile of
    w = workloads.block_sparse(mask, 320, seed=12)
    q = void.quantize_void_tensor(w.a)
    bq, bs = void.quantize_cols_int8(w.b)
    M, N = q.shape[0], 320
    slots = mode == "slots"
    for out_dtype in (torch.float16, torch.float32):
        full = void.void_spmm_int8(q, bq, bs, out_dtype=out_dtype)
        shards = [void.shard_void_tensor(q, strategy, world, r) for r in range(world)]
        assert sum(d.n_local_blocks for d in shards) == q.n_blocks
        states, bufs = [], []
        for d in shards:
            st0 = vr.build_state(d, N, out_dtype, mode=mode,
                                 scratch=vr.Scratch(torch.zeros(1, dtype=torch.uint8, device="cuda"), [0], 0, 0, 0))
            rows_max = max(e - s for s, e in st0.ranges)
            acc, ctr_off, out_off, total = vr._layout(rows_max, st0.n_chunks, st0.np, N, full.element_size(), world if slots else 0)
            buf = torch.zeros(total, dtype=torch.uint8, device="cuda")
            st0.scratch = vr.Scratch(buf, [], acc, ctr_off, out_off, None, slots)
            states.append(st0)
            bufs.append(buf)
        ptrs = [b_.data_ptr() for b_ in bufs]
        # which ranks hold tiles of which tile row (what contributors() gathers over the process group)
        contrib_all = torch.zeros(states[0].packed.nbr, dtype=torch.int32, device="cuda")
        for r, st0 in enumerate(states):
            contrib_all |= ((st0.packed.row_ptr[1:] - st0.packed.row_ptr[:-1]) > 0).to(torch.int32) << r
        contrib_all = contrib_all.to(torch.uint8)
        for call, order in enumerate((list(range(world)), list(reversed(range(world))))):
            sc = states[0].scratch
            parts = []
            if slots:
                for b_ in bufs:
                    b_[call * sc.acc_bytes:(call + 1) * sc.acc_bytes].fill_(0x5A)   # stale slots must not matter where a rank contributes
                for r in order:
                    vr.launch_reduce(states[r], bq, None, 1.0, ptrs, world, slot_set=call)
                for r, (s, e) in enumerate(states[0].ranges):
                    out_r = torch.full((max(e - s, 0) * 32, N), float("nan"), dtype=out_dtype, device="cuda")
                    vr.reduce_owned_rows(states[r], ptrs[r] + call * sc.acc_bytes, contrib_all[s:e].contiguous(), r, world, bs, 1.0, out_r)
                    parts.append(out_r[:max(min(e * 32, M) - s * 32, 0)])
            else:
                for b_ in bufs:
                    b_[sc.out_off:].fill_(0xFF)                   # stale rows of C must be overwritten
                for r in order:
                    vr.launch_reduce(states[r], bq, bs, 1.0, ptrs, world)
                for r, (s, e) in enumerate(states[0].ranges):
                    rows = max(min(e * 32, M) - s * 32, 0)
                    parts.append(bufs[r][sc.out_off: sc.out_off + rows * N * full.element_size()].view(out_dtype).view(rows, N))
                    torch.cuda.synchronize()
                    assert not bufs[r][:sc.out_off].any()           # accumulators and counters back at zero
            torch.cuda.synchronize()
            void.check_device_status()
            assert torch.equal(torch.cat(parts), full), (strategy, world, out_dtype, order, mode)


def test_sharded_workload_shape_vs_oracle():
    """The multi-GPU workload's shape (2048 x 2048 block grid at 95 %, N = 1024: eight panels, four chunks and about
    a hundred tiles per tile row): the shard of rank 3 of 8 against the oracle on sampled tile rows, first and last
    of the shard included - int32 accumulators bit for bit, fp16 output within 1e-3."""
    world, rank, N = 8, 3, 1024
    shard, (start, end), nnz = workloads.sharded_int8(world_size=world, rank=rank, seed=0)
    assert (start, end) == (768, 1024) and shard.shape == (256 * 32, 65536)
    g = torch.Generator(device="cuda").manual_seed(5)
    bq = torch.randint(-127, 128, (65536, N), dtype=torch.int8, device="cuda", generator=g)
    bs = torch.rand(N, device="cuda", generator=g) * 0.02 + 0.001
    acc = torch.empty(256 * 32, N, dtype=torch.int32, device="cuda")
    out = void.void_spmm_int8(shard, bq, bs, out_dtype=torch.float16, acc_out=acc)
    fast = void.void_spmm_int8(shard, bq, bs, out_dtype=torch.float16)       # the launch the benchmark times
    void.check_device_status()
    assert torch.equal(out, fast)
    rng = np.random.default_rng(0)
    sample = sorted(set([0, 255] + rng.choice(256, 32, replace=False).tolist()))
    rows_np, cols_np = shard.block_rows.cpu().numpy(), shard.block_cols.cpu().numpy()
    bs_np = bs.cpu().numpy()
    for r in sample:
        idx = np.nonzero(rows_np == r)[0]
        assert len(idx) > 50
        order = idx[np.argsort(cols_np[idx])]                      # the row's tiles by block column
        vals = shard.values[torch.from_numpy(order).cuda()].cpu().numpy()
        sc = shard.scales[torch.from_numpy(order).cuda()].cpu().numpy()
        # only the block rows of B the tile row touches, renumbered 0, 1, 2 ... (the oracle sees a [32, n * 32] matrix)
        take = (torch.from_numpy(cols_np[order].astype(np.int64)).cuda()[:, None] * 32 + torch.arange(32, device="cuda")).reshape(-1)
        b_sub = bq[take].cpu().numpy()
        zero_rows = np.zeros(len(order), dtype=np.int32)
        sub_cols = np.arange(len(order), dtype=np.int32)
        sub_shape = (32, len(order) * 32)
        ref_acc = vo.spmm_int8_acc(vals, zero_rows, sub_cols, sub_shape, b_sub)
        assert np.array_equal(acc[r * 32:(r + 1) * 32].cpu().numpy(), ref_acc[:32]), r
        ref = vo.spmm_int8(vals, sc, zero_rows, sub_cols, sub_shape, b_sub, col_scale=bs_np)
        got = out[r * 32:(r + 1) * 32].float().cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max(), r
