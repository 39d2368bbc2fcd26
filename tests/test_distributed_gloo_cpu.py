"""Host-side logic of the sharded SpMM with two gloo ranks on CPU: ROW_WISE ranges, the broadcast
of B from rank 0, the optional all_gather of the row shards.  The local product, which only exists
as a CUDA kernel, is replaced by the CPU oracle for this test (test infrastructure, never the
product path)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs():
    from oracle import void_oracle as vo
    rng = np.random.default_rng(21)
    nbr, nbc, n = 9, 6, 40                       # 9 tile rows over 2 ranks: 5 + 4 (ragged last shard)
    mask = rng.random((nbr, nbc)) < 0.5
    mask[3] = False
    rows, cols = np.nonzero(mask)
    order = np.argsort(vo.morton_encode_batch(rows, cols))
    rows, cols = rows[order].astype(np.int32), cols[order].astype(np.int32)
    vals = rng.standard_normal((len(rows), 32, 32)).astype(np.float32)
    q, s = vo.quantize_int8_tiles(vals)
    b = rng.standard_normal((nbc * 32, n)).astype(np.float32)
    bq, bs = vo.quantize_int8_cols(b)
    return (nbr * 32 - 7, nbc * 32), rows, cols, q, s, bq, bs


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import void_b200 as void
        from void_b200 import distributed as vd
        from oracle import void_oracle as vo
        shape, rows, cols, q, s, bq, bs = _inputs()
        a = void.Int8VOIDTensor(torch.from_numpy(q), torch.from_numpy(s), torch.zeros(len(rows), dtype=torch.int8),
                                torch.from_numpy(rows), torch.from_numpy(cols), shape, (32, 32), len(rows),
                                void.IntQuantConfig())
        d = void.shard_void_tensor(a)             # world size and rank from the process group
        assert d.world_size == world and d.rank == rank
        assert d.local_row_range == ((0, 5) if rank == 0 else (5, 9))
        # B lives on rank 0 only; the other rank receives it
        b_t = torch.from_numpy(bq) if rank == 0 else torch.zeros_like(torch.from_numpy(bq))
        s_t = torch.from_numpy(bs) if rank == 0 else torch.zeros_like(torch.from_numpy(bs))
        b_t, s_t = void.broadcast_b(b_t, src=0, scales=s_t)
        assert np.array_equal(b_t.numpy(), bq) and np.array_equal(s_t.numpy(), bs)

        def oracle_local(local, b, b_scale, out_dtype, out=None):
            c = vo.spmm_int8(local.values.numpy(), local.scales.numpy(), local.block_rows.numpy(),
                             local.block_cols.numpy(), local.shape, b.numpy(), col_scale=b_scale.numpy())
            c = torch.from_numpy(c)
            if out is not None:
                out.copy_(c)
                return out
            return c
        vd._local_spmm = oracle_local
        shard = void.distributed_void_spmm(d, b_t, b_scale=s_t, gather_output=False)
        full = void.distributed_void_spmm(d, b_t, b_scale=s_t)            # all_gather, like the reference
        ref = vo.spmm_int8(q, s, rows, cols, shape, bq, col_scale=bs)
        lo, hi = d.local_row_range
        assert np.array_equal(shard.numpy()[:min(hi * 32, shape[0]) - lo * 32], ref[lo * 32:hi * 32])
        assert full.shape == (shape[0], bq.shape[1]) and np.array_equal(full.numpy(), ref)
        # first product with B arriving in column panels (ragged last panel): same shard, and B ends up everywhere
        b2 = torch.from_numpy(bq).clone() if rank == 0 else torch.zeros_like(torch.from_numpy(bq))
        s2 = torch.from_numpy(bs).clone() if rank == 0 else torch.zeros_like(torch.from_numpy(bs))
        shard2, b2 = void.broadcast_spmm_overlapped(d, b2, s2, src=0, panel_cols=16)
        assert np.array_equal(b2.numpy(), bq) and np.array_equal(s2.numpy(), bs)
        assert shard2.shape == shard.shape and np.array_equal(shard2.numpy(), shard.numpy())
        # tile-balanced row ranges: shards of unequal height are gathered into the same full result
        db = void.shard_void_tensor(a, balance="nnz")
        assert db.row_ranges[0][0] == 0 and db.row_ranges[-1][1] == 9 and db.row_ranges[0][1] == db.row_ranges[1][0]
        full_b = void.distributed_void_spmm(db, b_t, b_scale=s_t)
        assert np.array_equal(full_b.numpy(), ref)
        # COLUMN_WISE / BLOCK_WISE of a floating tensor: local partial products of the whole C, summed by all_reduce
        # (the reference's route, void/distributed.py:252-267); the shards together give the unsharded product
        vals32 = (q.astype(np.float32) * s[:, None, None]).astype(np.float32)
        af = void.VOIDTensor(torch.from_numpy(vals32), torch.from_numpy(rows), torch.from_numpy(cols),
                             torch.zeros(len(rows), dtype=torch.int64), shape, (32, 32), 0, len(rows), 0.5)
        bf = torch.from_numpy(bq.astype(np.float32))

        def oracle_fp(local, b, b_scale, out_dtype, out=None):
            return torch.from_numpy(vo.spmm_fp(local.values.numpy(), local.block_rows.numpy(), local.block_cols.numpy(),
                                               local.shape, b.numpy())[:local.shape[0]])
        vd._local_spmm = oracle_fp
        want = vo.spmm_fp(vals32, rows, cols, shape, bf.numpy())[:shape[0]]
        for strat in (void.ShardingStrategy.COLUMN_WISE, void.ShardingStrategy.BLOCK_WISE):
            dc = void.shard_void_tensor(af, strat)
            got = void.distributed_void_spmm(dc, bf)
            assert got.shape == want.shape and np.allclose(got.numpy(), want, rtol=1e-5, atol=1e-3), strat
        ret[rank] = "ok"
    except Exception as e:  # pragma: no cover - surfaced through ret
        ret[rank] = repr(e)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_broadcast_gather():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


def test_sharding_single_process_defaults():
    import void_b200 as void
    shape, rows, cols, q, s, bq, bs = _inputs()
    a = void.Int8VOIDTensor(torch.from_numpy(q), torch.from_numpy(s), torch.zeros(len(rows), dtype=torch.int8),
                            torch.from_numpy(rows), torch.from_numpy(cols), shape, (32, 32), len(rows),
                            void.IntQuantConfig())
    d = void.shard_void_tensor(a)                 # no process group: world 1, rank 0
    assert d.world_size == 1 and d.rank == 0 and d.local_row_range == (0, 9)
    assert torch.equal(d.local_tensor.values, a.values) and d.n_local_blocks == len(rows)
    with pytest.raises(ValueError):
        void.shard_void_tensor(a, strategy="diagonal")
