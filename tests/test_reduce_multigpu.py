"""The sharded products over NCCL on two or more GPUs of one box, one process per GPU (skipped with fewer).

ROW_WISE: row shards and the reference's all_gather of them.  COLUMN_WISE / BLOCK_WISE: the sum over ranks inside
the SpMM kernel (partial int32 tiles added into the owning rank's accumulator over NVLink, last arriver finishes
the row), called twice in a row on different B.  Every result must equal the unsharded product on the same GPU
bit for bit.  No rank leaves early, nothing waits on another GPU inside a kernel, NVLS is off.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    import datetime
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    try:
        import void_b200 as void
        from void_b200 import workloads
        mask = workloads.uniform_mask(37, 29, 0.75, seed=31)
        mask[11] = False
        w = workloads.block_sparse(mask, 384, seed=31, device=dev)
        q = void.quantize_void_tensor(w.a)
        g = torch.Generator(device="cpu").manual_seed(99)
        b_list = [w.b, torch.randn(w.b.shape, generator=g).to(dev)]
        quant = [void.quantize_cols_int8(b) for b in b_list]
        notes = []
        for strategy in (void.ShardingStrategy.ROW_WISE, void.ShardingStrategy.COLUMN_WISE, void.ShardingStrategy.BLOCK_WISE):
            d = void.shard_void_tensor(q, strategy)
            assert d.world_size == world and d.rank == rank
            for out_dtype in (torch.float16, torch.float32):
                for bq, bs in quant:
                    want = void.void_spmm_int8(q, bq, bs, out_dtype=out_dtype)
                    full = void.distributed_void_spmm(d, bq, b_scale=bs, out_dtype=out_dtype)
                    assert full.shape == want.shape and torch.equal(full, want), (strategy, out_dtype, "gathered")
                    shard = void.distributed_void_spmm(d, bq, b_scale=bs, out_dtype=out_dtype, gather_output=False)
                    if strategy != void.ShardingStrategy.ROW_WISE:      # the single-kernel form with atomic adds as well
                        from void_b200.reduce import fused_reduce_spmm
                        again = fused_reduce_spmm(d, bq, bs, out_dtype, mode="atomic")
                        assert torch.equal(again, shard), (strategy, out_dtype, "atomic form")
                    s, e = d.owner_ranges()[rank]
                    rows = min(e * 32, q.shape[0]) - s * 32
                    assert torch.equal(shard[:rows], want[s * 32:s * 32 + rows]), (strategy, out_dtype, "shard")
            torch.cuda.synchronize()
            void.check_device_status()
            notes.append(strategy.value)
        # tile-balanced row ranges gather to the same result
        db = void.shard_void_tensor(q, balance="nnz")
        bq, bs = quant[0]
        assert torch.equal(void.distributed_void_spmm(db, bq, b_scale=bs, out_dtype=torch.float16),
                           void.void_spmm_int8(q, bq, bs, out_dtype=torch.float16))
        dist.barrier()
        ret[rank] = "ok " + ",".join(notes)
    except Exception as e:  # pragma: no cover - surfaced through ret
        import traceback
        ret[rank] = "".join(traceback.format_exception(type(e), e, e.__traceback__))[-1500:]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_products_over_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(str(v).startswith("ok") for v in dict(ret).values()) and len(ret) == world, dict(ret)
