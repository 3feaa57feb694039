"""Multi-GPU host logic on CPU: the shard plan, and a world_size-2 gloo run of
shard -> per-rank attention (the CPU oracle stands in for the GPU kernels) -> gather."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from inference_engine_b200.sharding import gather_outputs, plan_shards


def test_plan_is_balanced_and_deterministic():
    rng = np.random.default_rng(4)
    lens = np.exp(rng.uniform(np.log(512), np.log(32768), 2048)).astype(int)  # log-uniform contexts, as in the sharded benchmark
    for world in (1, 2, 4, 8):
        plan = plan_shards(lens, world)
        assert sorted(i for ids in plan.local for i in ids) == list(range(len(lens)))
        assert all(plan.owner[i] == r for r, ids in enumerate(plan.local) for i in ids)
        assert plan.imbalance() < 1.002
        assert plan_shards(lens, world).local == plan.local
    assert plan_shards([], 4).imbalance() == 1.0


def _worker(rank, world, port, lens, seed, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from tests import helpers as H

        plan = plan_shards(lens, world)
        mine = plan.local[rank]
        rng = np.random.default_rng(seed)  # same inputs on every rank, each computes only its shard
        q = H.randn_bf16(rng, len(lens), H.HQ, H.D)
        pages = sum((n + 15) // 16 for n in lens) + 1
        table = H.random_block_table(rng, lens, 16, pages)
        cache = H.random_filled_cache(rng, pages, 16, gauss=True)
        cached = np.array([n - 1 for n in lens], np.int32)
        local = O.decode_attention(q[mine], cache, cached[mine], table[mine], len(mine), H.D ** -0.5)
        full = gather_outputs(torch.from_numpy(local), plan, rank)
        if rank == 0:
            want = O.decode_attention(q, cache, cached, table, len(lens), H.D ** -0.5)
            ret["ok"] = bool(np.array_equal(full.numpy(), want))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_gather():
    lens = [300, 17, 129, 64, 1, 450, 33]
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, 29533, lens, 9, ret), nprocs=2, join=True)
        assert ret.get("ok") is True
