"""The sharded step's host logic on two CPU ranks (gloo): ownership, flat views, gather."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

SHAPES = [(40, 24), (24,), (8, 8, 3), (100,), (16, 64)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pylo_b200.zero import ShardedStep

        gen = torch.Generator().manual_seed(7)
        params = [torch.nn.Parameter(torch.randn(s, generator=gen)) for s in SHAPES]
        before = [p.detach().clone() for p in params]
        shard = ShardedStep(params)
        assert all(torch.equal(p.detach(), b) for p, b in zip(params, before)), "values must survive the re-pointing"
        assert sorted(i for r in range(world) for i in range(len(SHAPES)) if shard.owner[i] == r) == list(range(len(SHAPES)))
        with torch.no_grad():  # every rank "steps" only what it owns
            for i in shard.owned:
                params[i].add_(float(i + 1))
        shard.gather()
        for i, (p, b) in enumerate(zip(params, before)):
            assert torch.allclose(p.detach(), b + float(i + 1)), f"tensor {i} not gathered on rank {rank}"
        # the scalar all-reduce the global-norm clip needs
        t = torch.tensor([float(sum(p.detach().pow(2).sum() for i, p in enumerate(params) if i in shard.owned))])
        dist.all_reduce(t)
        total = float(sum(p.detach().pow(2).sum() for p in params))
        assert abs(t.item() - total) < 1e-3 * total
        out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_sharded_step_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results
