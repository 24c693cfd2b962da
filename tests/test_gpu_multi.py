"""Two ranks on two GPUs: the sharded step (whole-tensor ownership + parameter all-gather) gives the same
parameters as one process that owns everything.  Skipped when fewer than two GPUs are visible."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases

# ranks that disagree on the order of collectives should end the test, not sit out the default ten minutes
PG_TIMEOUT = datetime.timedelta(seconds=90)

pytestmark = pytest.mark.gpu

SHAPES = [(96, 64), (64,), (64, 160), (160,), (40, 40), (8, 6, 5), (40,)]
CASE = dict(shapes=SHAPES, init_seed=21, init_scale=0.05, grad_seed=22, grad_scale=0.2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _build(family, params_or_shard, sharded):
    from pylo_b200 import models, optim
    from pylo_b200.zero import sharded_optimizer

    torch.manual_seed(0)
    if family == "adafaclo":
        cls, kw = optim.AdafacLO_CUDA, dict(lr=1e-2, network=models.MetaMLP(39, 32, 1))
    elif family == "elo_celo2":
        cls, kw = optim.ELO_CELO2_CUDA, dict(lr=1e-2, network=models.CELO2MLP())   # clip_grad on by default
    else:
        rnn, mlp = models.VeLORNN(lstm_hidden_size=32), models.VeLOMLP()
        with torch.no_grad():
            for name, p in mlp.named_parameters():
                if name.endswith("_") or "_." in name:
                    p.mul_(0.05)
        cls, kw = optim.VeLO_CUDA, dict(lr=10.0, num_steps=100, rnn=rnn, mlp=mlp)
    return sharded_optimizer(cls, params_or_shard, **kw) if sharded else cls(params_or_shard, **kw)


def _worker(rank, world, port, family, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=PG_TIMEOUT)
    try:
        from pylo_b200.zero import ShardedStep

        loss = lambda t: torch.tensor(cases.velo_loss(t), device=dev)
        # sharded run
        params = [torch.nn.Parameter(v.to(dev)) for v in cases.init_values(CASE)]
        shard = ShardedStep(params)
        opt = _build(family, shard, True)
        for t in (1, 2, 3):
            grads = cases.grads_at(CASE, t)
            for i in shard.owned:
                params[i].grad = grads[i].to(dev)
            opt.step(loss(t)) if family == "velo" else opt.step()
            shard.gather()
        torch.cuda.synchronize()
        # the same three steps with everything on this rank
        ref = [torch.nn.Parameter(v.to(dev)) for v in cases.init_values(CASE)]
        opt1 = _build(family, ref, False)
        for t in (1, 2, 3):
            for p, g in zip(ref, cases.grads_at(CASE, t)):
                p.grad = g.to(dev)
            opt1.step(loss(t)) if family == "velo" else opt1.step()
        torch.cuda.synchronize()
        worst = max(float((a.detach() - b.detach()).abs().max()) for a, b in zip(params, ref))
        moved = max(float((b.detach().cpu() - v).abs().max()) for b, v in zip(ref, cases.init_values(CASE)))
        out.put((rank, "ok" if worst <= 1e-6 * max(1.0, moved / 1e-3) and moved > 0 else f"diff {worst} moved {moved}"))
    except Exception as e:  # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


def _staged_worker(rank, world, port, out, lone_tensor=None):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=PG_TIMEOUT)
    try:
        from pylo_b200 import models, optim
        from pylo_b200.zero import StagedShardedStep

        # lone_tensor: a single tensor, so that the second rank owns nothing and still has to start every gather
        shapes = [(72, 48)] if lone_tensor else SHAPES + [(72, 48), (48, 72), (30, 200)]
        case = dict(CASE, shapes=shapes)
        shard = StagedShardedStep(shapes, dev, blocks=3, init_scale=0.05, seed=4)
        start = [p.detach().clone() for p in shard.params]

        def make(params):
            torch.manual_seed(0)
            if lone_tensor == "celo2":
                return optim.CELO2_CUDA(params, lr=1e-2, clip_grad=True, network=models.CELO2MLP())
            return optim.AdafacLO_CUDA(params, lr=1e-2, network=models.MetaMLP(39, 32, 1))

        opt = make(shard.param_groups())
        opt.after_group = shard.after_group
        opt._sharded = True
        for t in (1, 2, 3):
            grads = cases.grads_at(case, t)
            for i in shard.owned:
                shard.params[i].grad = grads[i].to(dev)
            opt.step()
            shard.finish()
        torch.cuda.synchronize()
        ref = [torch.nn.Parameter(v.clone()) for v in start]
        opt1 = make(ref)
        for t in (1, 2, 3):
            for p, g in zip(ref, cases.grads_at(case, t)):
                p.grad = g.to(dev)
            opt1.step()
        torch.cuda.synchronize()
        same = all(torch.equal(a.detach(), b.detach()) for a, b in zip(shard.params, ref))
        moved = any(not torch.equal(a.detach(), b) for a, b in zip(ref, start))
        out.put((rank, "ok" if same and moved else f"same={same} moved={moved}"))
    except Exception:  # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


def _fused_worker(rank, world, port, family, out, multicast=False, push="stores"):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=PG_TIMEOUT)
    try:
        from pylo_b200 import models, optim
        from pylo_b200.zero import FusedShardedStep

        shapes = SHAPES + [(72, 48), (300, 260)]
        case = dict(CASE, shapes=shapes)
        shard = FusedShardedStep(shapes, dev, init_scale=0.05, seed=4, multicast=multicast, push=push)
        if multicast is None and not shard.multicast_base:
            out.put((rank, "no-multicast"))
            return
        start = [p.detach().clone() for p in shard.params]
        loss = lambda t: torch.tensor(cases.velo_loss(t), device=dev)

        def make(params, sharded):
            torch.manual_seed(0)
            if family == "adafaclo":
                return optim.AdafacLO_CUDA(params, lr=1e-2, network=models.MetaMLP(39, 32, 1))
            rnn, mlp = models.VeLORNN(lstm_hidden_size=32), models.VeLOMLP()
            with torch.no_grad():
                for name, p in mlp.named_parameters():
                    if name.endswith("_") or "_." in name:
                        p.mul_(0.05)
            kw = dict(all_shapes=shapes, owned=shard.owned) if sharded else {}
            return optim.VeLO_CUDA(params, lr=10.0, num_steps=100, rnn=rnn, mlp=mlp, **kw)

        if push == "copies" and family == "adafaclo":   # two param groups: each one's range leaves when it is enqueued
            opt = make(shard.param_groups(groups=2), True)
            opt.after_group = shard.after_group
        else:                                            # no hook: finish() pushes the whole owned region
            opt = make([shard.params[i] for i in shard.owned], True)
        for t in (1, 2, 3):
            grads = cases.grads_at(case, t)
            for i in shard.owned:
                shard.params[i].grad = grads[i].to(dev)
            opt.step(loss(t)) if family == "velo" else opt.step()
            shard.finish()
        torch.cuda.synchronize()
        ref = [torch.nn.Parameter(v.clone()) for v in start]
        opt1 = make(ref, False)
        for t in (1, 2, 3):
            for p, g in zip(ref, cases.grads_at(case, t)):
                p.grad = g.to(dev)
            opt1.step(loss(t)) if family == "velo" else opt1.step()
        torch.cuda.synchronize()
        same = all(torch.equal(a.detach(), b.detach()) for a, b in zip(shard.params, ref))
        moved = any(not torch.equal(a.detach(), b) for a, b in zip(ref, start))
        # the consolidated checkpoint equals what the single-process optimizer saves
        from pylo_b200.zero import consolidate_state_dict

        full = consolidate_state_dict(opt, shard, dst=0)
        if rank == 0:
            want = opt1.state_dict()["state"]
            for i, st in want.items():
                for name, v in st.items():
                    got = full["state"][i][name]
                    if torch.is_tensor(v):
                        same = same and torch.equal(got, v.detach().cpu())
                    else:
                        same = same and got == v
        out.put((rank, "ok" if same and moved else f"same={same} moved={moved}"))
    except Exception:  # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()[-800:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("family", ["adafaclo", "velo"])
def test_two_rank_fused_exchange_is_bit_identical(family):
    """Parameters reach the other rank as peer stores from the apply kernels (no all-gather)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_worker, args=(r, 2, port, family, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


@pytest.mark.parametrize("family", ["adafaclo", "velo"])
def test_two_rank_copy_pushed_exchange_is_bit_identical(family):
    """The kernels store locally; every param group's range is copied into the peer's buffer on a side stream."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_worker, args=(r, 2, port, family, out, False, "copies")) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


@pytest.mark.parametrize("family", ["adafaclo", "velo"])
def test_two_rank_fused_multicast_exchange_is_bit_identical(family):
    """The same through the NVLink switch's multicast mapping of the buffer: one multimem store per value."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_worker, args=(r, 2, port, family, out, None)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    if any(msg == "no-multicast" for _, msg in results):
        pytest.skip("the symmetric memory offers no multicast address on this system")
    assert all(msg == "ok" for _, msg in results), results


def test_two_rank_staged_step_with_overlapped_gathers_is_bit_identical():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_staged_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


@pytest.mark.parametrize("family", ["adafaclo", "celo2"])
def test_rank_that_owns_nothing_still_takes_part(family):
    """One tensor, two ranks: the second rank's optimizer has only empty param groups, and must still start every
    block's all-gather (and the all-reduce of the gradient norm) in the same order as the first."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_staged_worker, args=(r, 2, port, out, family)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


@pytest.mark.parametrize("family", ["adafaclo", "elo_celo2", "velo"])
def test_two_rank_sharded_step_matches_single_process(family):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, family, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def _intake_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=PG_TIMEOUT)
    try:
        from pylo_b200 import models, optim
        from pylo_b200.zero import FusedShardedStep

        shapes = SHAPES + [(72, 48), (300, 260)]
        case = dict(CASE, shapes=shapes)
        shard = FusedShardedStep(shapes, dev, init_scale=0.05, seed=4, multicast=False)
        start = [p.detach().clone() for p in shard.params]
        shard.attach_grads()
        torch.manual_seed(0)
        opt = optim.AdafacLO_CUDA([shard.params[i] for i in shard.owned], lr=1e-2, network=models.MetaMLP(39, 32, 1))
        torch.manual_seed(0)
        ref = [torch.nn.Parameter(v.clone()) for v in start]
        opt1 = optim.AdafacLO_CUDA(ref, lr=1e-2, network=models.MetaMLP(39, 32, 1))
        same = True
        for t in (1, 2, 3):
            # every replica computed its own gradients of ALL tensors (here: seeded per rank and step) ...
            shard.zero_grads()
            for p, g in zip(shard.params, cases.grads_at(dict(case, grad_seed=CASE["grad_seed"] + 10 * rank), t)):
                p.grad.copy_(g.to(dev))
            # ... the reference answer: all-reduce everything, then every rank would slice out what it owns
            summed = [p.grad.detach().clone() for p in shard.params]
            for v in summed:
                dist.all_reduce(v)
            shard.reduce_scatter_grads()
            same = same and all(torch.equal(shard.params[i].grad, summed[i]) for i in shard.owned)
            opt.step()
            shard.finish()
            for p, g in zip(ref, summed):
                p.grad = g
            opt1.step()
        torch.cuda.synchronize()
        same = same and all(torch.equal(a.detach(), b.detach()) for a, b in zip(shard.params, ref))
        out.put((rank, "ok" if same else "sharded step fed by the reduce-scatter differs from the all-reduce run"))
    except Exception:  # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()[-800:]))
    finally:
        dist.destroy_process_group()


def test_two_rank_reduce_scatter_gradient_intake_is_bit_identical():
    """Gradients reach their owners by one reduce-scatter over the flat layout; the step that follows equals the
    step of one process fed with all-reduced gradients, bit for bit."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_intake_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results
