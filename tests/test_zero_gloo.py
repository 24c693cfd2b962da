"""The sharded step's host logic on two CPU ranks (gloo): ownership, flat views, gather."""

import datetime
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
        # gradient intake: every replica has its own gradients of ALL tensors; after the reduce-scatter each rank holds
        # the sum for the tensors it owns, bit-identical to an all-reduce followed by a slice
        shard.attach_grads()
        g = torch.Generator().manual_seed(100 + rank)
        mine = [torch.randn(sh, generator=g) for sh in SHAPES]
        for p, v in zip(params, mine):
            p.grad.copy_(v)                       # what a backward pass would leave
        summed = [v.clone() for v in mine]
        for v in summed:
            dist.all_reduce(v)
        shard.reduce_scatter_grads()
        for i in shard.owned:
            assert torch.equal(params[i].grad, summed[i]), f"gradient of tensor {i} on rank {rank}"
        shard.zero_grads()
        assert all(float(p.grad.abs().max()) == 0.0 for p in params)
        assert all(p.grad.data_ptr() == shard.flat_grad[off:].data_ptr() for p, off in zip(params, shard.offsets))
        out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        out.put((rank, traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


def _worker_staged(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pylo_b200 import zero

        # the [block][rank] layout of the staged step, without its CUDA streams: layout and intake only
        shard = zero.StagedShardedStep.__new__(zero.StagedShardedStep)
        shard.pg, shard.world, shard.rank, shard.blocks = None, world, rank, 2
        shard.owner, shard.block, shard.offsets, shard.subs = zero.partition_blocks(SHAPES, world, 2)
        shard.base = [sum(shard.subs[:b]) * world for b in range(2)]
        shard.flat = torch.zeros(sum(shard.subs) * world)
        shard.params = [torch.nn.Parameter(shard.flat[o:o + zero._numel(sh)].view(sh)) for o, sh in zip(shard.offsets, SHAPES)]
        shard.owned = [i for i, r in enumerate(shard.owner) if r == rank]
        shard.attach_grads()
        g = torch.Generator().manual_seed(200 + rank)
        mine = [torch.randn(sh, generator=g) for sh in SHAPES]
        for p, v in zip(shard.params, mine):
            p.grad.copy_(v)
        summed = [v.clone() for v in mine]
        for v in summed:
            dist.all_reduce(v)
        shard.reduce_scatter_grads(average=True)
        for i in shard.owned:
            assert torch.equal(shard.params[i].grad, summed[i] / world), f"gradient of tensor {i} on rank {rank}"
        out.put((rank, "ok"))
    except Exception:  # pragma: no cover
        import traceback
        out.put((rank, traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


def _worker_idle_rank(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        from pylo_b200 import zero

        # one tensor, two ranks, three blocks: the second rank owns nothing, yet has to start every block's gather
        shapes = [(72, 48)]
        shard = zero.StagedShardedStep(shapes, "cpu", blocks=3, init_scale=0.05, seed=4)
        groups = shard.param_groups()
        counts = [None] * world
        dist.all_gather_object(counts, (len(groups), [closes for _, closes in shard._group_info]))
        assert counts[0] == counts[1], f"ranks disagree on their param groups: {counts}"
        assert len(groups) == 3 and (rank == 0 or all(len(g["params"]) == 0 for g in groups))
        before = shard.flat.clone()
        # what an optimizer does: update the tensors of a group (if any), then call the hook - for EVERY group
        for gi, g in enumerate(groups):
            for p in g["params"]:
                p.data.add_(1.0)
            shard.after_group(gi)
        shard.finish()
        flats = [torch.empty_like(shard.flat) for _ in range(world)]
        dist.all_gather(flats, shard.flat)
        assert torch.equal(flats[0], flats[1]), "the ranks' parameter buffers differ after the gathers"
        assert torch.equal(shard.params[0].detach(), before[shard.offsets[0]:shard.offsets[0] + 72 * 48].view(72, 48) + 1.0)
        out.put((rank, "ok"))
    except Exception:  # pragma: no cover
        import traceback
        out.put((rank, traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


def test_rank_without_tensors_starts_every_gather_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_idle_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def test_staged_layout_gradient_intake_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_staged, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


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
