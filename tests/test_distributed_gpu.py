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
