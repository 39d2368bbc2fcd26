"""Host logic of the sharding modes on CPU tensors: the product's shard_void_tensor against the reference's
own output (tests/golden/shard_small.npz), the tile-balanced row ranges, and the ownership / segment table of
the fused reduce (no GPU, no collective: index arithmetic only)."""
import os

import numpy as np
import pytest
import torch

import void_b200 as void
from void_b200 import distributed as vd

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _tensor_from_fixture(g):
    n = len(g["block_rows"])
    values = torch.zeros(n, 32, 32)
    values[:, 0, 0] = torch.arange(n, dtype=torch.float32)          # every tile carries its stored position
    return void.VOIDTensor(values=values, block_rows=torch.from_numpy(g["block_rows"]),
                           block_cols=torch.from_numpy(g["block_cols"]), morton_codes=torch.zeros(n, dtype=torch.int64),
                           shape=tuple(int(x) for x in g["shape"]), tile_size=(32, 32), nnz_original=n, n_blocks=n,
                           density=0.5)


@pytest.mark.parametrize("strategy", list(void.ShardingStrategy))
def test_shard_void_tensor_matches_reference_output(strategy):
    g = np.load(os.path.join(GOLDEN, "shard_small.npz"))
    vt = _tensor_from_fixture(g)
    nbr = vt.block_grid[0]
    for world in (int(w) for w in g["worlds"]):
        for rank in range(world):
            tag = "%s_w%d_r%d_" % (strategy.value, world, rank)
            d = void.shard_void_tensor(vt, strategy, world, rank)
            lt = d.local_tensor
            meta = [int(x) for x in g[tag + "meta"]]
            assert np.array_equal(lt.values[:, 0, 0].numpy().astype(np.int64), g[tag + "ids"]), tag
            assert np.array_equal(lt.block_rows.numpy(), g[tag + "rows"]), tag
            assert np.array_equal(lt.block_cols.numpy(), g[tag + "cols"]), tag
            assert lt.n_blocks == meta[6] and tuple(d.global_shape) == tuple(meta[7:9])
            ref_rows, ref_cols, ref_shape = meta[0:2], meta[2:4], meta[4:6]
            if ref_rows[0] <= nbr and ref_cols[0] <= vt.block_grid[1]:
                assert list(d.local_row_range) == ref_rows and list(d.local_col_range) == ref_cols, tag
                assert list(lt.shape) == ref_shape, tag
            else:
                # a rank past the end: the reference reports start > end and a negative local extent; here the
                # empty range is clamped to the end of the grid and the extent is zero
                assert lt.n_blocks == 0 and min(lt.shape) == 0


def test_shards_of_every_strategy_partition_the_tiles():
    g = np.load(os.path.join(GOLDEN, "shard_small.npz"))
    vt = _tensor_from_fixture(g)
    for strategy in void.ShardingStrategy:
        for world in (1, 2, 3, 5, 8):
            ids = [void.shard_void_tensor(vt, strategy, world, r).local_tensor.values[:, 0, 0] for r in range(world)]
            assert torch.equal(torch.sort(torch.cat(ids)).values, torch.arange(vt.n_blocks, dtype=torch.float32))


def test_tile_balanced_row_ranges_on_power_law_rows():
    """Equal row counts leave a power-law matrix badly balanced; ranges cut by tile count stay within 10 %."""
    from void_b200 import workloads
    mask = workloads.zipf_mask(512, 512, 1.5, 512, 15.36, seed=0)
    rows, cols = np.nonzero(mask)
    block_rows = torch.from_numpy(rows.astype(np.int32))
    counts = np.bincount(rows, minlength=512)
    for world in (2, 4, 8):
        ranges = vd.balanced_row_ranges(block_rows, 512, world)
        assert ranges[0][0] == 0 and ranges[-1][1] == 512
        assert all(ranges[k][1] == ranges[k + 1][0] for k in range(world - 1))
        per_rank = np.array([counts[a:b].sum() for a, b in ranges], dtype=np.float64)
        equal = np.array([counts[a:b].sum() for a, b in (vd.row_range(512, world, r) for r in range(world))], dtype=np.float64)
        assert per_rank.sum() == counts.sum()
        assert per_rank.max() / per_rank.mean() <= 1.1, (world, per_rank)
        assert per_rank.max() <= equal.max()


def test_balanced_shard_keeps_order_and_rebases():
    g = np.load(os.path.join(GOLDEN, "shard_small.npz"))
    vt = _tensor_from_fixture(g)
    seen = []
    for rank in range(3):
        d = void.shard_void_tensor(vt, void.ShardingStrategy.ROW_WISE, 3, rank, balance="nnz")
        start, end = d.local_row_range
        assert d.row_ranges[rank] == (start, end)
        ids = d.local_tensor.values[:, 0, 0].long()
        assert (torch.diff(ids) > 0).all()
        assert torch.equal(d.local_tensor.block_rows.long() + start, vt.block_rows[ids].long())
        assert d.local_tensor.shape == ((end - start) * 32, vt.shape[1])
        seen.append(ids)
    assert torch.equal(torch.sort(torch.cat(seen)).values, torch.arange(vt.n_blocks))


def test_reduce_plan_covers_every_row_once_and_names_its_owner():
    """Plan of the in-kernel reduction: every (tile row, chunk) appears once per rank, with the owner the
    ROW_WISE range of the row, a scratch index inside the owner's rows, and this rank's tile range of the row."""
    from void_b200.reduce import reduce_segments
    g = np.load(os.path.join(GOLDEN, "shard_small.npz"))
    vt = _tensor_from_fixture(g)
    nbr, nbc = vt.block_grid
    for world in (1, 2, 3, 8):
        ranges = [vd.row_range(nbr, world, r) for r in range(world)]
        for strategy in (void.ShardingStrategy.COLUMN_WISE, void.ShardingStrategy.BLOCK_WISE):
            tiles_seen = 0
            for rank in range(world):
                d = void.shard_void_tensor(vt, strategy, world, rank)
                rows = d.local_tensor.block_rows.long()
                row_ptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(torch.bincount(rows, minlength=nbr), 0)]).int()
                for n_chunks, n_cta in ((1, 4), (3, 7), (2, 1000)):
                    segs, ptr, used = reduce_segments(row_ptr, n_chunks, world, rank, ranges, n_cta)
                    segs = segs.view(-1, 8).long()
                    assert segs.shape[0] == nbr * n_chunks and ptr[0] == 0 and ptr[-1] == nbr * n_chunks
                    assert (torch.diff(ptr.long()) >= 0).all() and ptr.numel() == used + 1
                    keys = segs[:, 0] * n_chunks + segs[:, 1]
                    assert torch.equal(torch.sort(keys).values, torch.arange(nbr * n_chunks))
                    for row, chunk, t0, t1, nseg, owner, me, ctr in segs.tolist():
                        s, e = ranges[owner]
                        assert s <= row < e and nseg == world and me == rank
                        assert ctr == (row - s) * n_chunks + chunk and 0 <= ctr < (e - s) * n_chunks
                        assert (t0, t1) == (int(row_ptr[row]), int(row_ptr[row + 1]))
                    if world > 1:       # the first row a rank visits belongs to the next rank
                        assert segs[0, 5].item() == (rank + 1) % world or ranges[(rank + 1) % world][0] >= nbr
                tiles_seen += int(row_ptr[-1])
            assert tiles_seen == vt.n_blocks


def test_tile_list_with_repeated_or_out_of_range_coordinates_is_rejected():
    """The device index builder skips coordinates outside the grid and counts a repeated pair once; the host
    check that follows it compares the indexed count with the listed one."""
    from void_b200.format import check_tile_index
    check_tile_index(torch.tensor([0, 2, 2, 5], dtype=torch.int32), 5)            # consistent: accepted
    with pytest.raises(ValueError, match="1 of 5 tiles"):
        check_tile_index(torch.tensor([0, 2, 2, 4], dtype=torch.int32), 5)
