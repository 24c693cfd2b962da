#!/usr/bin/env python
"""Benchmark of the learned-optimizer step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload llama3_8b|gpt2_medium|vit_b16|celo2_4096|mlp_784] [--optimizer adafaclo|...]

One "step" is one ``optimizer.step()`` over every parameter tensor of the
workload (plus, with more than one GPU, the exchange of the updated
parameters).  Tensors are owned ZeRO-1 style by one rank each, so the total
work is fixed as N grows (strong scaling).  Prints ONE JSON line on rank 0.

The headline line is AdafacLO over the Llama-3-8B parameter shapes.  With the
default workload the line also carries ``extra_configs``: the other benchmark
configurations (VeLO over the GPT-2-medium shapes, CELO2 on one 4096 x 4096
weight, ELO_CELO2 over the ViT-B/16 shapes, CELO2 over the Llama shapes), each
with Newton-Schulz off and on where the family has it, measured after the
headline in the same process.

``--impl reference`` times the CPU restatement of the reference's step
(oracle/pylo_oracle.py) on the host cores of the box, on a bounded sample of the
same workload; it is the only place besides the ``cpu_baseline`` and
``reference_cuda`` legs where this script executes anything under oracle/, and
it does not load the CUDA library of this package.
"""

import argparse
import copy
import datetime
import gc
import json
import os
import subprocess
import sys
import threading
import time
import types

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "optimizer_step_params_per_sec"
UNIT = "params/s"
# compulsory HBM bytes per parameter of a whole step: g, p, m(3), v read once; p, m(3), v written once
STEP_BYTES = {"adafaclo": 44, "elo": 44, "velo": 44, "celo2": 56, "elo_celo2": 56}
# compulsory bytes per parameter of the apply sweep alone (reads g, p, m(3), v; writes p or the raw step)
APPLY_BYTES = 28
B_BYTES = 40  # state_moments sweep: reads g, p, m(3), v; writes m(3), v
# DRAM bytes per element (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels: CONSTANTS taken
# from ncu captures of a 4096 x 4096 case, not measured in this run; traffic grows in proportion to the elements
NCU_TRAFFIC_PER_ELEM = {"k_apply_adafac_cols": 27.58, "k_apply_adafac_tc": 27.44}
# TF32 / fp16 multiply-adds the tensor-core apply kernels issue per parameter (products x N x K, M = the element)
TC_ISSUED_FMA_PER_PARAM = {"3xtf32": (9 + 12 + 1) * 32 * 8}   # 22 products of N = 32, K = 8 per element row


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="llama3_8b")
    ap.add_argument("--optimizer", default="adafaclo", choices=sorted(STEP_BYTES))
    ap.add_argument("--layers", type=int, default=None, help="llama3_8b only: number of transformer layers (default 32)")
    ap.add_argument("--no-orthogonalize", action="store_true", help="celo2 family: skip Newton-Schulz")
    ap.add_argument("--ns-precision", default="3xtf32", choices=["fp32", "3xtf32"],
                    help="celo2 family: Newton-Schulz products on the tensor cores by this library's kernel (operands split "
                         "into TF32 high and low parts), or as fp32 torch.matmul (the reference's arithmetic; a library call)")
    ap.add_argument("--mlp-precision", default="3xtf32", choices=["fp32", "3xtf32"],
                    help="adafaclo / elo: the network's hidden layers as scalar fp32 FMAs, or as tensor-core products of "
                         "operands split into two TF32 parts (fp32-faithful: hi x hi + hi x lo + lo x hi)")
    ap.add_argument("--blocks", type=int, default=8, help="N>1: stages whose parameter all-gathers overlap the next stage")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "copy", "staged"],
                    help="N>1: how updated parameters reach the other ranks (fused: peer stores from the apply kernels; "
                         "copy: one device-to-device copy per param group and peer on side streams; staged: NCCL "
                         "all-gathers per block)")
    ap.add_argument("--no-multicast", action="store_true",
                    help="N>1, fused exchange: one store per peer instead of one multimem store through the switch")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other benchmark configurations (extra_configs)")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip the timing of the reference's own CUDA kernels")
    ap.add_argument("--cpu-sample-steps", type=int, default=3)
    return ap.parse_args(argv)


def import_without_native_library():
    """Make ``pylo_b200.workloads`` and ``pylo_b200.models`` importable WITHOUT running the package's
    ``__init__`` (which loads libpylo_b200.so): the CPU reference arm needs only shape lists and the seeded
    meta-networks, and must not map this package's CUDA library into its process."""
    if "pylo_b200" not in sys.modules:
        pkg = types.ModuleType("pylo_b200")
        pkg.__path__ = [os.path.join(ROOT, "pylo_b200")]
        sys.modules["pylo_b200"] = pkg


def workload_shapes(args):
    from pylo_b200 import workloads as W

    if args.workload == "llama3_8b":
        return W.llama3_8b(args.layers or 32)
    return W.WORKLOADS[args.workload]()


def grad_spec(args):
    return {"llama3_8b": (1e-4, "iid"), "llama3_block": (1e-4, "iid"), "gpt2_medium": (1e-3, "outliers"), "vit_b16": (1e-3, "iid"),
            "celo2_4096": (1.0, "rowlognormal"), "mlp_784": (1e-3, "iid")}[args.workload]


def seeded_networks(kind):
    from pylo_b200 import models

    torch.manual_seed(0)
    if kind in ("adafaclo", "elo"):
        return models.MetaMLP(39, 32, 1)
    if kind in ("celo2", "elo_celo2"):
        return models.CELO2MLP()
    rnn, mlp = models.VeLORNN(), models.VeLOMLP()
    with torch.no_grad():
        for name, p in mlp.named_parameters():
            if name.endswith("_") or "_." in name:
                p.mul_(0.05)  # the banks are N(0,1) by default and get multiplied by 100 when mixed
    return rnn, mlp


def is_embedding_shape(shape):
    """Token embedding / lm head: routed to the AdamW branch in the CELO2 family."""
    return len(shape) == 2 and shape[0] > 32768


def build_optimizer(args, shard, params):
    from pylo_b200 import optim

    k = args.optimizer
    if k == "velo":
        rnn, mlp = seeded_networks(k)
        return optim.VeLO_CUDA(params, lr=1e-3, num_steps=10000, rnn=rnn, mlp=mlp, process_group=shard.pg,
                               all_shapes=[tuple(p.shape) for p in shard.params], owned=shard.owned)
    from pylo_b200.zero import FusedShardedStep

    # several param groups even on one GPU: the optimizer runs them in order, so the end-to-end leg can
    # let group k compute while the gradients of group k+1 are still arriving from the host
    groups = shard.param_groups(groups=args.blocks) if isinstance(shard, FusedShardedStep) else shard.param_groups()
    if k == "adafaclo":
        opt = optim.AdafacLO_CUDA(groups, lr=1e-3, step_mult=0.01, exp_mult=0.001, network=seeded_networks(k),
                                  mlp_precision=args.mlp_precision)
    elif k == "elo":
        opt = optim.ELO_CUDA(groups, lr=1e-3, weight_decay=0.1, clip_grad=True, network=seeded_networks(k),
                             mlp_precision=args.mlp_precision)
    else:
        cls = optim.CELO2_CUDA if k == "celo2" else optim.ELO_CELO2_CUDA
        opt = cls(shard.param_groups(is_embedding_shape), lr=1e-3, weight_decay=0.1,
                  orthogonalize=not args.no_orthogonalize, network=seeded_networks(k), ns_precision=args.ns_precision)
    opt._sharded, opt.process_group = shard.world > 1, shard.pg
    opt.after_group = shard.after_group
    return opt


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample_shapes(args, shapes):
    """A bounded sample of the workload for the CPU legs: one mid-sized matrix and one vector of it."""
    mats = sorted({s for s in shapes if len(s) >= 2}, key=lambda s: abs(s[0] * s[1] - 4_194_304) if len(s) == 2 else 1e18)
    vecs = sorted({s for s in shapes if len(s) == 1})
    sample = [mats[0]] + ([vecs[0]] if vecs else [])
    return sample


def run_cpu_oracle(args, shapes, steps, warmup=1):
    """Time the oracle's step on the host cores; returns (params/s, cores, sample description)."""
    from oracle import pylo_oracle as O
    from pylo_b200 import workloads as W

    torch.set_num_threads(os.cpu_count() or 1)
    sample = cpu_sample_shapes(args, shapes)
    gscale, gkind = grad_spec(args)
    gen = torch.Generator().manual_seed(1)
    params = [torch.randn(s, generator=gen) * 0.02 for s in sample]
    grads = [torch.randn(s, generator=gen) * gscale for s in sample]
    k = args.optimizer
    if k in ("adafaclo", "elo"):
        net = seeded_networks(k)
        o = O.AdafacLOOracle(net.flat_weights(), lr=1e-3, elo=(k == "elo"), weight_decay=0.1 if k == "elo" else 0.0,
                             clip_grad=(k == "elo"))
        step = lambda: o.step(params, grads)
    elif k in ("celo2", "elo_celo2"):
        net = seeded_networks(k)
        o = O.CELO2Oracle(net.flat_weights(), lr=1e-3, weight_decay=0.1, orthogonalize=not args.no_orthogonalize,
                          shared_adam=(k == "elo_celo2"), clip_grad=(k == "elo_celo2"),
                          adam_lr_mult=20.0 if k == "elo_celo2" else 1.0)
        step = lambda: o.step(params, grads)
    else:
        rnn, mlp = seeded_networks(k)
        o = O.VeLOOracle(O.rnn_weights_from_module(rnn), O.bank_from_module(mlp), sample, lr=1e-3, num_steps=10000)
        step = lambda: o.step(params, grads, 1.0)
    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    n = W.total_params(sample)
    mean = sum(times) / len(times)
    desc = f"{' + '.join(str(s) for s in sample)} of the workload, {steps} step(s) after {warmup} warm-up"
    return n / mean, torch.get_num_threads(), desc, mean


def config_of(args, shapes, n_gpus):
    from pylo_b200 import workloads as W

    gscale, gkind = grad_spec(args)
    return {
        "workload": f"{args.optimizer} step over {args.workload} parameter shapes ({len(shapes)} tensors, "
                    f"{W.total_params(shapes) / 1e9:.3f} G fp32 params), ZeRO-1 whole-tensor ownership",
        "optimizer": args.optimizer, "shapes": args.workload, "tensors": len(shapes),
        "params": W.total_params(shapes), "grads": f"randn*{gscale} ({gkind}), one buffer per distinct shape",
        "orthogonalize": (not args.no_orthogonalize) if "celo2" in args.optimizer else None,
        "newton_schulz": (None if "celo2" not in args.optimizer or args.no_orthogonalize else
                          ("k_gemm_tn_3xtf32 (this library, tcgen05)" if args.ns_precision == "3xtf32" else "torch.matmul fp32 (library)")),
        "mlp_precision": args.mlp_precision if args.optimizer in ("adafaclo", "elo") else None,
        "cache": "inputs larger than L2 (no flush needed)" if W.total_params(shapes) * 24 / max(n_gpus, 1) > 2e9
                 else "L2 flushed between steps by writing a 512 MiB buffer",
        "parallelism": f"zero1x{n_gpus}", "exchange": getattr(args, "exchange_used", "none"),
        "gather_blocks": (args.blocks if getattr(args, "exchange_used", "") == "staged" and args.optimizer != "velo" else 1),
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import_without_native_library()
    shapes = workload_shapes(args)
    steps = max(1, args.steps)
    value, cores, desc, mean = run_cpu_oracle(args, shapes, steps, warmup=max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(args, shapes, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def replica_checksum(flat):
    """Order-independent, exact checksums of a rank's whole flat parameter buffer: the sum of its bit patterns
    (as integers) and the sum of their squares modulo 2^63, taken in chunks so that nothing large is allocated."""
    s1 = torch.zeros((), dtype=torch.int64, device=flat.device)
    s2 = torch.zeros((), dtype=torch.int64, device=flat.device)
    bits = flat.view(torch.int32)
    step = 1 << 26
    for lo in range(0, bits.numel(), step):
        c = bits[lo:lo + step].to(torch.int64)
        s1 += c.sum()
        s2 += (c * c).remainder(2147483647).sum()
    return torch.stack([s1, s2])


def ranks_agree(ok, world, dev):
    """True if ``ok`` holds on every rank (one tiny all-reduce; at one rank just ``ok``)."""
    if world == 1:
        return bool(ok)
    import torch.distributed as dist

    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(int(flag.item()))


def measure(args, dev, world, rank, local, headline):
    """One configuration on the current process group: returns the JSON line (rank 0) or None."""
    import torch.distributed as dist

    from pylo_b200 import workloads as W
    from pylo_b200.zero import FusedShardedStep, ShardedStep, StagedShardedStep

    shapes = workload_shapes(args)
    total = W.total_params(shapes)
    gscale, gkind = grad_spec(args)

    # memory guard: never drive the box out of memory (the previous configuration's optimizer sits in reference
    # cycles through its hooks until the collector has run)
    gc.collect()
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info()
    state_bytes = 16 if args.optimizer not in ("celo2", "elo_celo2") else 20
    need = total * 4 + (total / world) * (state_bytes + 1) * 1.02 + 4e9
    why = None
    if need > free * 0.97:
        why = f"workload needs ~{need / 1e9:.0f} GB per GPU, {free / 1e9:.0f} GB free: refusing to run"
    # the ranks decide together: one rank that skipped a configuration while the others ran its collectives would
    # leave them waiting for it
    if not ranks_agree(why is None, world, dev):
        raise MemoryError(why or "another rank has too little free memory for this workload: refusing to run")

    exchange = args.exchange
    if exchange == "auto":
        exchange = "fused" if args.optimizer in ("adafaclo", "elo", "velo") else "staged"
    if world == 1:
        exchange = "none"
    shard = None
    if exchange in ("fused", "copy") or (world == 1 and args.optimizer in ("adafaclo", "elo")):
        # N>1: parameters reach the other ranks as peer stores from the apply kernels; N=1: plain flat buffer
        ok, why = 1, ""
        try:
            shard = FusedShardedStep(shapes, dev, init_scale=0.02, seed=1, multicast=False if args.no_multicast else None,
                                     push="copies" if exchange == "copy" else "stores")
        except Exception as e:  # symmetric memory unavailable on this box: fall back to NCCL gathers
            ok, why = 0, repr(e)
        if world > 1:
            flag = torch.tensor([ok], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = int(flag.item())
        if not ok:
            if rank == 0:
                print(f"fused exchange unavailable ({why or 'another rank failed'}); using NCCL gathers", file=sys.stderr)
            shard, exchange = None, "staged"
            torch.cuda.empty_cache()
    if shard is not None:
        pass
    elif args.optimizer == "velo":  # its LSTM needs every tensor's statistics before any tensor is applied
        shard = ShardedStep.from_shapes(shapes, dev, init_scale=0.02, seed=1)
    else:                      # NCCL all-gathers per block, overlapped with the next block's kernels
        shard = StagedShardedStep(shapes, dev, blocks=min(args.blocks, 4), init_scale=0.02, seed=1)
    if exchange == "fused" and getattr(shard, "multicast_base", 0):
        exchange = "fused-multicast"
    if exchange == "copy":
        exchange = "copies-per-group"
    args.exchange_used = exchange
    owned = shard.owned
    params = [shard.params[i] for i in owned]
    why = None
    try:
        pool = W.make_grad_pool([shapes[i] for i in owned], gscale, dev, seed=2 + rank, kind=gkind)
        for p in params:
            p.grad = pool[tuple(p.shape)]
        opt = build_optimizer(args, shard, params)
    except Exception as e:
        why = f"{type(e).__name__}: {e}"
    if not ranks_agree(why is None, world, dev):
        raise RuntimeError(why or "another rank could not set this configuration up")
    owned_n = sum(p.numel() for p in params)
    velo = args.optimizer == "velo"
    loss = torch.tensor(1.0, device=dev)
    flush = None
    if total * 24 / world <= 2e9:
        flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def one_step():
        if flush is not None:
            flush.fill_(1)
        if velo:
            opt.step(loss)
            shard.gather()   # all-gather, or (fused exchange) the one-element all-reduce that orders the peer stores
        else:
            opt.step()       # starts each block's all-gather as soon as the block's kernels are enqueued
            shard.finish()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def plans():
        out = []
        for v in getattr(opt, "_plans", {}).values():
            out.append(v[1]["lo"] if isinstance(v[1], dict) else v[1])
        if getattr(opt, "_plan", None):
            out.append(opt._plan[1]["plan"])
        return [p for p in out if p is not None]

    for _ in range(max(args.warmup, 3)):
        one_step()
    barrier()
    for pl in plans():
        pl.enable_profile(True)
        pl.launch_count = 0
    extra_launches0 = getattr(opt, "extra_launches", 0)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    ev[0].record()
    for _ in range(args.steps):
        one_step()
    ev[1].record()
    barrier()
    elapsed_ms = ev[0].elapsed_time(ev[1])
    if hasattr(opt, "check_status"):
        opt.check_status()  # raises if a bounded wait of the tensor-core kernel ran out during the timed steps
    clocks = sampler.stop() if rank == 0 else None
    phase = {}
    launches = getattr(opt, "extra_launches", 0) - extra_launches0
    for pl in plans():
        for k, v in pl.phase_times().items():
            phase.setdefault(pl.KERNEL_OF.get(k, k), []).extend(v)
        launches += pl.launch_count
        pl.enable_profile(False)
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = total / (ms_per_step * 1e-3)

    # ---- end to end: gradients arrive from pinned host memory, a probe of the result goes back
    e2e = None
    if headline and not args.no_e2e:
        pinned = {s: torch.empty(s, dtype=torch.float32).pin_memory() for s in pool}
        for s, buf in pinned.items():
            buf.copy_(pool[s])
        probe_idx = torch.tensor([shard.offsets[i] for i in owned], device=dev)
        h2d = sum(p.numel() for p in params) * 4
        d2h = len(owned) * 4

        copy_stream = torch.cuda.Stream(device=dev)
        group_params = [list(g["params"]) for g in opt.param_groups] if not velo else [params]
        events = [torch.cuda.Event() for _ in group_params]

        def e2e_step():
            # gradients of group k+1 arrive from pinned host memory while group k computes
            copy_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(copy_stream):
                for gi, plist in enumerate(group_params):
                    for p in plist:
                        p.grad.copy_(pinned[tuple(p.shape)], non_blocking=True)
                    events[gi].record(copy_stream)
            if velo:
                torch.cuda.current_stream().wait_event(events[0])
            one_step()
            return shard.flat.index_select(0, probe_idx).cpu()

        if not velo:
            opt.before_group = lambda gi: torch.cuda.current_stream().wait_event(events[gi])
        e2e_step()
        barrier()
        ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        t0 = time.perf_counter()
        ev2[0].record()
        for _ in range(args.steps):
            e2e_step()
        ev2[1].record()
        barrier()
        wall = (time.perf_counter() - t0) * 1e3
        te = torch.tensor([max(ev2[0].elapsed_time(ev2[1]), wall)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.item()) / args.steps
        hb = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(hb)
        e2e = {"value": total / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(hb[0].item()), "d2h_bytes_per_step": int(hb[1].item())}
        opt.before_group = None

    # ---- every rank must now hold the same parameters, bit for bit
    replica = None
    if world > 1:
        barrier()
        mine = replica_checksum(shard.flat)
        allsums = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allsums, mine)
        replica = {"ranks": world, "equal": bool(all(torch.equal(a, allsums[0]) for a in allsums)),
                   "what": "sum of bit patterns and sum of their squares (mod 2^31-1) of every rank's whole flat "
                           "parameter buffer after the last step"}

    line = None
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
        mean = lambda xs: sum(xs) / max(len(xs), 1)
        phase_ms = {k: mean(v) for k, v in phase.items()}
        phase_share = {k: sum(v) for k, v in phase.items()}
        dominant = max(phase_share, key=phase_share.get) if phase_share else None
        lo_elems = sum(pl.total_elems for pl in plans())
        n_launch = max(len(phase.get(dominant, [])), 1)
        per_launch_elems = lo_elems * args.steps / n_launch if dominant else 0
        kbytes = B_BYTES if dominant == "k_state_moments" else (4 if dominant == "k_rowcol_fast" else
                                                                 (APPLY_BYTES if dominant and dominant.startswith("k_apply") else 0))
        achieved = per_launch_elems * kbytes / (phase_ms.get(dominant, 1e9) * 1e-3) / 1e9 if dominant else 0.0
        roofline = {
            "bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": f"{peak_src} (MEASURED_PEAKS.json hbm_gbs)",
            "traffic": (NCU_TRAFFIC_PER_ELEM[dominant] * per_launch_elems if dominant in NCU_TRAFFIC_PER_ELEM else None),
            "traffic_note": "constant: dram bytes per element from an ncu capture of a 4096x4096 case, times the elements "
                            "of one launch (not measured in this run)",
            "algorithmic_bytes_per_param": kbytes, "avg_launch_ms": phase_ms.get(dominant),
            "phase_ms_per_launch": phase_ms, "phase_share": {k: v / max(sum(phase_share.values()), 1e-9) for k, v in phase_share.items()},
            "step": {"algorithmic_bytes_per_param": STEP_BYTES[args.optimizer],
                     "achieved": owned_n * STEP_BYTES[args.optimizer] / (ms_per_step * 1e-3) / 1e9,
                     "frac": owned_n * STEP_BYTES[args.optimizer] / (ms_per_step * 1e-3) / 1e9 / peak},
        }
        if args.optimizer in ("adafaclo", "elo") and dominant == "k_apply_adafac_tc":
            per_param = TC_ISSUED_FMA_PER_PARAM[args.mlp_precision]
            issued = per_launch_elems * per_param * 2 / (phase_ms[dominant] * 1e-3)
            roofline["tensor"] = {"network_fma_per_param": 1600, "issued_fma_per_param": per_param,
                                  "operands": "tf32", "products_per_128_params": 22,
                                  "issued_tflops": issued / 1e12,
                                  "network_fp32_equiv_tflops": per_launch_elems * 3200 / (phase_ms[dominant] * 1e-3) / 1e12}
        elif args.optimizer in ("adafaclo", "elo") and dominant in ("k_apply", "k_apply_adafac_cols") and clocks and clocks.get("sm_mhz"):
            # the apply sweep of the 39-32-32-2 network is bound by fp32 FMA issue, not by HBM
            fma = per_launch_elems * 1600 / (phase_ms[dominant] * 1e-3)
            peak_fma = 148 * 128 * clocks["sm_mhz"] * 1e6
            roofline["fp32_fma"] = {"fma_per_param": 1600, "achieved_tfma": fma / 1e12,
                                    "peak_tfma_at_sampled_clock": peak_fma / 1e12, "frac": fma / peak_fma}
        cpu = None
        if headline and not args.no_cpu_baseline and world == 1:
            v, cores, desc, _ = run_cpu_oracle(args, shapes, args.cpu_sample_steps)
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        cfg = config_of(args, shapes, world)
        if replica is not None:
            cfg["replica_check"] = replica
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        }
    ok = replica is None or replica["equal"]
    # free this configuration's memory before the next one is built
    del opt, shard, params, pool
    torch.cuda.empty_cache()
    return line, ok


# the other benchmark configurations, measured after the headline: (name, workload, optimizer, extra arguments, timed steps)
EXTRA_CONFIGS = [
    ("velo/gpt2_medium", "gpt2_medium", "velo", [], 50),
    ("celo2/celo2_4096/ns_off", "celo2_4096", "celo2", ["--no-orthogonalize"], 100),
    ("celo2/celo2_4096/ns_on", "celo2_4096", "celo2", [], 30),
    ("celo2/celo2_4096/ns_on_torch_matmul", "celo2_4096", "celo2", ["--ns-precision=fp32"], 20),
    ("elo_celo2/vit_b16/ns_off", "vit_b16", "elo_celo2", ["--no-orthogonalize"], 100),
    ("elo_celo2/vit_b16/ns_on", "vit_b16", "elo_celo2", [], 30),
    ("elo_celo2/vit_b16/ns_on_torch_matmul", "vit_b16", "elo_celo2", ["--ns-precision=fp32"], 20),
    ("celo2/llama3_8b/ns_off", "llama3_8b", "celo2", ["--no-orthogonalize"], 3),
    ("celo2/llama3_8b/ns_on", "llama3_8b", "celo2", [], 1),
]


def compact(name, line):
    r = line["roofline"]
    return {"name": name, "workload": line["config"]["workload"], "ms_per_step": line["ms_per_step"], "steps": line["steps"],
            "value": line["value"], "unit": UNIT, "orthogonalize": line["config"]["orthogonalize"],
            "newton_schulz": line["config"].get("newton_schulz"),
            "exchange": line["config"]["exchange"], "cache": line["config"]["cache"],
            "replica_check": line["config"].get("replica_check"),
            "roofline": {"step_frac": r["step"]["frac"], "step_bytes_per_param": r["step"]["algorithmic_bytes_per_param"],
                         "kernel": r["kernel"], "kernel_frac": r["frac"], "kernel_avg_launch_ms": r["avg_launch_ms"],
                         "phase_share": r["phase_share"]},
            "gpu_launches": line["gpu_launches"], "clocks": line["clocks"]}


def run_b200(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # a short limit: the longest step of any configuration here takes seconds; if ranks ever disagree on the
        # order of collectives the run should end, not sit out the default ten minutes on eight GPUs
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    try:
        line, ok = measure(args, dev, world, rank, local, headline=True)
    except MemoryError as e:
        raise SystemExit(str(e))
    all_ok = ok
    default_run = args.workload == "llama3_8b" and args.optimizer == "adafaclo" and args.layers is None
    if default_run and not args.no_extra:
        extras = []
        for name, workload, optimizer, more, steps in EXTRA_CONFIGS:
            sub = copy.copy(args)
            sub.workload, sub.optimizer, sub.steps, sub.warmup = workload, optimizer, steps, 3
            sub.no_orthogonalize = "--no-orthogonalize" in more
            sub.ns_precision = "fp32" if "--ns-precision=fp32" in more else "3xtf32"
            if workload == "llama3_8b" and world == 1:
                # 8.03 G parameters with the CELO2 family's 20 B/param of state do not fit one GPU: 16 of the 32 layers
                sub.layers = 16
                name += "/16_layers"
            try:
                sub_line, ok = measure(sub, dev, world, rank, local, headline=False)
                all_ok = all_ok and ok
                if rank == 0:
                    extras.append(compact(name, sub_line))
            except Exception as e:  # a configuration that cannot run here is reported, not fatal to the headline
                if rank == 0:
                    extras.append({"name": name, "error": f"{type(e).__name__}: {e}"[:300]})
                torch.cuda.empty_cache()
        if rank == 0:
            line["extra_configs"] = extras
    if rank == 0:
        if world == 1 and not args.no_reference_cuda:
            line["reference_cuda"] = run_reference_cuda(dev)
        emit(line)
    if world > 1:
        dist.destroy_process_group()
    if not all_ok:
        raise SystemExit("replica_check failed: the ranks' parameter buffers differ after the last step")


def run_reference_cuda(dev):
    """The reference's OWN CUDA kernels (built from its sources into oracle/_ref/ by oracle/build_ref.py) timed on
    this GPU next to this library, on a bounded sample: the "kernel to beat"."""
    probed = [os.path.join(ROOT, "oracle", "_ref", n + ".so") for n in ("cuda_lo", "celo2_cuda_kernel", "velo_cuda_kernel")]
    if not all(os.path.exists(p) for p in probed):
        return {"status": "unavailable", "why": "the reference's CUDA extensions were not built into oracle/_ref/",
                "probed": probed}
    try:
        from oracle import ref_cuda
        return ref_cuda.time_against_library(dev, seeded_networks)
    except Exception as e:
        return {"status": "unavailable", "why": f"{type(e).__name__}: {e}"[:300], "probed": probed}


def emit(line):
    """Print the result line on the real stdout (see main)."""
    sys.stdout.flush()
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = 1


def main():
    # Libraries below (NCCL among them) sometimes write banners to file descriptor 1.  The contract is ONE JSON
    # line on stdout, so descriptor 1 is pointed at stderr for the whole run and the line goes to a saved copy.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
