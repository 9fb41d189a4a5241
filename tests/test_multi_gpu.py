"""Two real GPUs, one process each (NCCL): every rank decodes its shard of a batch in its
own page pool; the gathered rows equal the single-GPU result bit for bit.  Skipped on
boxes with fewer than two GPUs (the world-size-2 gloo test covers the host logic on CPU)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    import attention_b200 as attn
    from attention_b200 import sharding, synth

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        w = synth.scaled("c5_skewed_bf16", batch=24, len_hi=6000)
        q, k, v, table, lens = synth.make_workload(w, seed=42)          # same global case everywhere
        shards = sharding.lpt_assign(lens.tolist(), world)
        local = sharding.extract_shard(q, k, v, table, lens, shards[rank], device=dev)
        mine = attn.gqa_decode(*local, chunk_tokens=512)
        biggest = max(len(s) for s in shards)
        padded = torch.zeros((biggest,) + tuple(mine.shape[1:]), dtype=mine.dtype, device=dev)
        padded[: mine.shape[0]] = mine
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded)                                  # harness only, not data path
        if rank == 0:
            parts = [p[: len(s)] for p, s in zip(parts, shards)]
            whole = sharding.scatter_outputs(parts, shards, w.batch)
            single = attn.gqa_decode(q.to(dev), k.to(dev), v.to(dev), table.to(dev), lens.to(dev),
                                     chunk_tokens=512)
            ret["equal"] = bool(torch.equal(whole, single))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_decode_is_bit_identical():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert ret["equal"] is True
