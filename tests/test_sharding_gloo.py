"""World-size-2 (and 3) run of the multi-GPU host path on CPU with the gloo backend.

Each rank takes its LPT shard of a workload, builds its own page pool and table,
computes its rows (with the CPU oracle standing in for the device kernels, which
need a GPU), and the rows are gathered and compared with the unsharded result.
Timing is reduced with MAX over ranks as the benchmark does.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gqa_oracle

from attention_b200 import sharding, synth


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        w = synth.scaled("c5_skewed_bf16", batch=10, len_hi=600)
        q, k, v, table, lens = synth.make_workload(w, seed=42)      # every rank: same global case
        shards = sharding.lpt_assign(lens.tolist(), world)
        local = sharding.extract_shard(q, k, v, table, lens, shards[rank])
        # local pool holds exactly this rank's pages, renumbered from 0
        used = int(((local[4].long() + w.block_size - 1) // w.block_size).sum())
        assert local[1].shape[0] == max(1, used)
        assert int(local[3].max()) == used - 1
        mine = gqa_oracle.gqa_decode_c(*local, threads=1)
        # gather variable-sized parts: pad to the largest shard
        biggest = max(len(s) for s in shards)
        padded = torch.zeros((biggest,) + tuple(mine.shape[1:]), dtype=torch.float32)
        padded[: mine.shape[0]] = mine.float()
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded)
        parts = [p[: len(s)].to(mine.dtype) for p, s in zip(parts, shards)]
        whole = sharding.scatter_outputs(parts, shards, w.batch)
        # max-over-ranks reduction used for timing
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        if rank == 0:
            ref = gqa_oracle.gqa_decode_c(q, k, v, table, lens, threads=1)
            ret["equal"] = bool(torch.equal(whole, ref))
            ret["tmax"] = float(t)
            ret["imbalance"] = sharding.load_imbalance(lens.tolist(), shards)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_decode_matches_unsharded_over_gloo(world):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert ret["equal"] is True
        assert ret["tmax"] == float(world)
        assert ret["imbalance"] < 1.35
