"""ZeRO-1 style sharding of the optimizer step across the GPUs of one box.

Every reduction of the learned-optimizer step is per tensor (row/column sums,
feature normalisers, the CELO2 tail, Newton-Schulz), so a rank that owns a
whole tensor needs nothing from the others to update it.  Ownership is
therefore whole-tensor: a deterministic longest-processing-time assignment by
cost.  Parameters live in one flat fp32 buffer laid out
``[rank 0's tensors | pad][rank 1's tensors | pad]...`` with equal-sized rank
regions; after the local step one in-place ``all_gather_into_tensor`` over NCCL
(NVLink / NVSwitch) makes every rank's copy complete again.  The global-norm
clip adds one scalar ``all_reduce``.

The reference has no distributed code; its documentation describes exactly this
scheme in prose (docs/concepts.rst:274-283).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

ALIGN = 64  # floats; every tensor starts on a 256-byte boundary inside the flat buffer


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def partition(shapes: Sequence[Tuple[int, ...]], world_size: int,
              cost: Optional[Callable[[Tuple[int, ...]], float]] = None) -> List[int]:
    """Owner rank of every tensor: greedy longest-processing-time, ties by index; deterministic."""
    cost = cost or (lambda s: float(_numel(s)))
    order = sorted(range(len(shapes)), key=lambda i: (-cost(shapes[i]), i))
    load = [0.0] * world_size
    owner = [0] * len(shapes)
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += cost(shapes[i])
    return owner


def flat_layout(shapes: Sequence[Tuple[int, ...]], owner: Sequence[int], world_size: int):
    """Offsets (in floats) of every tensor in the flat buffer and the per-rank region size."""
    used = [0] * world_size
    local = [0] * len(shapes)
    for i, s in enumerate(shapes):
        r = owner[i]
        local[i] = used[r]
        used[r] += (_numel(s) + ALIGN - 1) // ALIGN * ALIGN
    shard = max(max(used), ALIGN)
    offsets = [owner[i] * shard + local[i] for i in range(len(shapes))]
    return offsets, shard


def partition_blocks(shapes: Sequence[Tuple[int, ...]], world_size: int, blocks: int,
                     cost: Optional[Callable[[Tuple[int, ...]], float]] = None):
    """Owner rank and block of every tensor, for a step that is cut into ``blocks`` stages.

    Tensors are first balanced over the ranks (as :func:`partition`), then each rank's tensors over its
    blocks; the buffer is laid out ``[block][rank][tensors | pad]`` so that the parameters a stage updates
    form, over all ranks, one contiguous range that a single all-gather can fill while the next stage
    computes.  Returns (owner, block, offsets, subs) with ``subs[b]`` the size of one rank's cell in block b.
    """
    cost = cost or (lambda s: float(_numel(s)))
    owner = partition(shapes, world_size, cost)
    block = [0] * len(shapes)
    sizes = [(_numel(s) + ALIGN - 1) // ALIGN * ALIGN for s in shapes]
    per_rank = max(sum(sz for sz, o in zip(sizes, owner) if o == r) for r in range(world_size))
    # block capacities are the same on every rank: the first block is as large as the largest tensor
    # needs (a tensor cannot be split), the rest share what remains
    first = max(max(sizes), -(-per_rank // blocks))
    rest = -(-max(per_rank - first, 0) // max(blocks - 1, 1))
    caps = [first] + [rest] * (blocks - 1)
    for r in range(world_size):
        mine = sorted((i for i, o in enumerate(owner) if o == r), key=lambda i: (-sizes[i], i))
        fill = [0] * blocks
        for i in mine:  # first fit, largest first; what fits nowhere goes to the emptiest block
            fits = [b for b in range(blocks) if fill[b] + sizes[i] <= caps[b]]
            bsel = fits[0] if fits else min(range(blocks), key=lambda b: (fill[b] - caps[b], b))
            block[i] = bsel
            fill[bsel] += sizes[i]
    used = {}
    local = [0] * len(shapes)
    for i, s in enumerate(shapes):
        key = (block[i], owner[i])
        local[i] = used.get(key, 0)
        used[key] = local[i] + (_numel(s) + ALIGN - 1) // ALIGN * ALIGN
    subs = [max([used.get((b, r), 0) for r in range(world_size)] + [ALIGN]) for b in range(blocks)]
    base = [0] * blocks
    for b in range(1, blocks):
        base[b] = base[b - 1] + subs[b - 1] * world_size
    offsets = [base[block[i]] + owner[i] * subs[block[i]] + local[i] for i in range(len(shapes))]
    return owner, block, offsets, subs


class _GradIntake:
    """Gradient intake for a sharded step: data-parallel replicas reduce-scatter their gradients so that every rank
    receives exactly the gradients of the tensors it owns, already summed (docs/concepts.rst:274-283 describes the
    scheme; the reference ships no code for it).

    The gradients of ALL tensors live in one flat buffer with the parameters' layout, and every parameter's
    ``.grad`` is a view into it, so autograd accumulates straight into the buffer.  Because a rank's tensors are
    contiguous in that layout (per block, for the staged layout), one ``reduce_scatter_tensor`` per block leaves the
    summed gradients of the owned tensors in a rank-sized buffer; the owned parameters' ``.grad`` are then re-pointed
    at it, which is what the optimizer reads.  Nothing else crosses the links: compared with an all-reduce every
    rank receives 1/N of the bytes.
    """

    def _grad_segments(self):
        """[(offset of the segment in the flat buffer, size of one rank's cell)] - one segment per gather block."""
        return [(0, self.shard)]

    def attach_grads(self):
        """Allocate the flat gradient buffer and point every parameter's ``.grad`` into it (zeroed)."""
        self.flat_grad = torch.zeros(self.flat.numel(), dtype=torch.float32, device=self.flat.device)
        segs = self._grad_segments()
        self._grad_cells = [torch.zeros(cell, dtype=torch.float32, device=self.flat.device) for _, cell in segs]
        self._point_grads_at_flat()
        return self.flat_grad

    def _point_grads_at_flat(self):
        for p, off in zip(self.params, self.offsets):
            p.grad = self.flat_grad[off:off + p.numel()].view(p.shape)

    def zero_grads(self):
        """Before the next backward pass: zero the flat buffer and point every ``.grad`` back into it."""
        self.flat_grad.zero_()
        self._point_grads_at_flat()

    def reduce_scatter_grads(self, average: bool = False):
        """Sum (``average``: mean) the replicas' gradients; afterwards the ``.grad`` of every OWNED parameter is the
        reduced gradient.  The gradients of tensors owned elsewhere are left as this replica computed them."""
        for (start, cell), out in zip(self._grad_segments(), self._grad_cells):
            if self.world > 1:
                dist.reduce_scatter_tensor(out, self.flat_grad[start:start + self.world * cell], group=self.pg)
            else:
                out.copy_(self.flat_grad[start:start + cell])
            if average and self.world > 1:
                out.div_(self.world)
        segs = self._grad_segments()
        for i in self.owned:
            off = self.offsets[i]
            k = max(j for j, (start, _) in enumerate(segs) if start <= off)   # the segment this tensor lies in
            start, cell = segs[k]
            local = off - start - self.rank * cell
            p = self.params[i]
            p.grad = self._grad_cells[k][local:local + p.numel()].view(p.shape)


class ShardedStep(_GradIntake):
    """Flat parameter buffer + ownership + the post-step gather for one process group.

    ``params`` are ``nn.Parameter``s (or tensors) in a fixed global order that is
    identical on every rank; their ``.data`` is re-pointed into the flat buffer.
    ``owned`` lists the indices this rank updates; build the optimizer over
    ``[params[i] for i in owned]`` and call :meth:`gather` after ``optimizer.step()``.
    """

    def __init__(self, params: Sequence[torch.Tensor], process_group=None,
                 cost: Optional[Callable[[Tuple[int, ...]], float]] = None, copy_values: bool = True):
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.params = list(params)
        shapes = [tuple(p.shape) for p in self.params]
        self.owner = partition(shapes, self.world, cost)
        self.offsets, self.shard = flat_layout(shapes, self.owner, self.world)
        dev = self.params[0].device
        self.flat = torch.zeros(self.shard * self.world, dtype=torch.float32, device=dev)
        for p, off, s in zip(self.params, self.offsets, shapes):
            view = self.flat[off:off + _numel(s)].view(s)
            if copy_values:
                view.copy_(p.data)
            p.data = view
        self.owned = [i for i, r in enumerate(self.owner) if r == self.rank]

    @classmethod
    def from_shapes(cls, shapes: Sequence[Tuple[int, ...]], device, init_scale: float = 0.02, seed: int = 1,
                    process_group=None, cost=None) -> "ShardedStep":
        """Allocate the flat buffer first and create the parameters as seeded views into it
        (no second copy of the parameters ever exists)."""
        self = cls.__new__(cls)
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        shapes = [tuple(s) for s in shapes]
        self.owner = partition(shapes, self.world, cost)
        self.offsets, self.shard = flat_layout(shapes, self.owner, self.world)
        self.flat = torch.zeros(self.shard * self.world, dtype=torch.float32, device=device)
        gen = torch.Generator(device=device)
        self.params = []
        for i, (off, s) in enumerate(zip(self.offsets, shapes)):
            view = self.flat[off:off + _numel(s)].view(s)
            gen.manual_seed(seed * 1000003 + i)
            view.normal_(0.0, init_scale, generator=gen)
            self.params.append(torch.nn.Parameter(view, requires_grad=True))
        self.owned = [i for i, r in enumerate(self.owner) if r == self.rank]
        return self

    def my_region(self) -> torch.Tensor:
        return self.flat[self.rank * self.shard:(self.rank + 1) * self.shard]

    def gather(self, async_op: bool = False):
        """All-gather every rank's region in place; afterwards all ranks hold all updated parameters."""
        if self.world == 1:
            return None
        return dist.all_gather_into_tensor(self.flat, self.my_region(), group=self.pg, async_op=async_op)


def split_in_groups(params, groups: int):
    """Consecutive runs of ``params`` with similar numbers of elements, as optimizer param groups."""
    total = sum(p.numel() for p in params)
    out, cur, acc = [], [], 0
    for p in params:
        cur.append(p)
        acc += p.numel()
        if len(out) < groups - 1 and acc >= total * (len(out) + 1) / groups:
            out.append({"params": cur})
            cur = []
    if cur or not out:   # a rank that owns nothing still gets one (empty) group: its hooks must run
        out.append({"params": cur})
    return out


class FusedShardedStep(_GradIntake):
    """Sharded step whose parameter exchange is fused into the apply kernels.

    The flat parameter buffer of every rank is allocated as symmetric memory, so each rank can address
    its peers' buffers directly.  The kernels that write a parameter store the new value into the
    owner's buffer and, with plain stores over NVLink, into the same offset of every other rank's
    buffer (``pylo_tensor_desc.p_peer``); no separate all-gather runs and no SMs are taken away from
    the apply sweep by a communication kernel.  :meth:`finish` is the only collective left: a
    one-element all-reduce that orders "all peers have finished writing" before the parameters are
    read again.  Supported by the AdafacLO / ELO and VeLO kernels (the CELO2 family writes its
    parameters in a separate tail kernel and keeps the NCCL gather of :class:`StagedShardedStep`).
    """

    def __init__(self, shapes: Sequence[Tuple[int, ...]], device, init_scale: float = 0.02, seed: int = 1,
                 process_group=None, cost=None, multicast: Optional[bool] = None, push: str = "stores"):
        """``multicast``: reach the peers through the NVLink switch's multicast mapping of the buffer (one
        ``multimem`` store per value, replicated by the switch) instead of one store per peer.  None: use it
        where the symmetric memory offers a multicast address, True: require it, False: never.

        ``push``: "stores" (the apply kernels store into the peers' buffers themselves) or "copies": the kernels
        store locally only, and once a param group's kernels are enqueued (:meth:`after_group`) the range of the
        buffer that group owns is copied into every peer's buffer with one device-to-device copy per peer, each
        on a stream of its own.  Those copies are the driver's (copy engines, no SMs) and keep NVLink busy while
        the next groups' sweeps - all of them, not only the apply sweeps - run."""
        if push not in ("stores", "copies"):
            raise ValueError("push must be 'stores' or 'copies'")
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        shapes = [tuple(s) for s in shapes]
        self.owner = partition(shapes, self.world, cost)
        self.offsets, self.shard = flat_layout(shapes, self.owner, self.world)
        n = self.shard * self.world
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            self.flat = symm.empty(n, dtype=torch.float32, device=device)
            self.handle = symm.rendezvous(self.flat, process_group if process_group is not None else dist.group.WORLD)
            bases = [int(b) for b in self.handle.buffer_ptrs]
            if bases[self.rank] != self.flat.data_ptr():
                raise RuntimeError("symmetric memory rendezvous returned an unexpected local address")
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            if multicast and not mc:
                raise RuntimeError("multicast=True, but the symmetric memory has no multicast address on this system")
            self.multicast_base = mc if multicast is not False else 0
        else:
            self.flat = torch.zeros(n, dtype=torch.float32, device=device)
            bases = [self.flat.data_ptr()]
            self.multicast_base = 0
        gen = torch.Generator(device=device)
        self.params = []
        for i, (off, s) in enumerate(zip(self.offsets, shapes)):
            view = self.flat[off:off + _numel(s)].view(s)
            gen.manual_seed(seed * 1000003 + i)
            view.normal_(0.0, init_scale, generator=gen)
            self.params.append(torch.nn.Parameter(view, requires_grad=True))
        self.owned = [i for i, r in enumerate(self.owner) if r == self.rank]
        self.push = push if self.world > 1 else "stores"
        self._group_ranges, self._pushed = [], False
        if self.push == "copies":
            peers = [r for r in range(self.world) if r != self.rank]
            self._peer_flat = [self.handle.get_buffer(r, (n,), torch.float32) for r in peers]
            self._copy_streams = [torch.cuda.Stream(device=device) for _ in peers]
        for i in self.owned if self.push == "stores" else []:  # where this tensor lives in every other rank's buffer
            if self.multicast_base:
                self.params[i]._pylo_peer_ptrs = [self.multicast_base + 4 * self.offsets[i]]
                self.params[i]._pylo_peer_multicast = True
            else:
                self.params[i]._pylo_peer_ptrs = [bases[r] + 4 * self.offsets[i] for r in range(self.world) if r != self.rank]
        self._token = torch.zeros(1, dtype=torch.float32, device=device)

    def param_groups(self, is_embedding=None, groups: int = 1):
        """The owned tensors as ``groups`` param groups of similar size, in buffer order (the optimizer
        runs its param groups one after the other, which lets a caller pipeline gradient arrival)."""
        out = split_in_groups([self.params[i] for i in self.owned], groups)
        index_of = {id(self.params[i]): i for i in self.owned}
        self._group_ranges = []
        for g in out:  # a group's tensors are consecutive in the owner's region: one contiguous range
            idx = [index_of[id(p)] for p in g["params"]]
            self._group_ranges.append((min(self.offsets[i] for i in idx), max(self.offsets[i] + self.params[i].numel() for i in idx))
                                      if idx else (0, 0))
        return out

    def _push_range(self, a: int, b: int):
        self._pushed = True
        if b <= a:
            return
        ev = torch.cuda.Event()
        ev.record()
        src = self.flat[a:b]
        for dst, stream in zip(self._peer_flat, self._copy_streams):
            with torch.cuda.stream(stream):
                stream.wait_event(ev)
                dst[a:b].copy_(src, non_blocking=True)
        self._pushed = True

    def after_group(self, gi: int):
        """Hook for the optimizer: param group ``gi`` is enqueued.  With ``push="copies"`` its range starts
        travelling to the peers now."""
        if self.push == "copies" and gi < len(self._group_ranges):
            self._push_range(*self._group_ranges[gi])

    def finish(self):
        """Order the peers' writes before the next read of the parameters: with ``push="copies"`` join the copy
        streams (pushing the whole owned region first if no hook ran this step), then one tiny all-reduce - a rank's
        contribution to it is enqueued behind its own stores or copies, so its completion here means every peer is
        done writing into this rank's buffer."""
        if self.world > 1:
            if self.push == "copies":
                if not self._pushed and self.owned:
                    a = min(self.offsets[i] for i in self.owned)
                    b = max(self.offsets[i] + self.params[i].numel() for i in self.owned)
                    self._push_range(a, b)
                cur = torch.cuda.current_stream()
                for stream in self._copy_streams:
                    cur.wait_stream(stream)
                self._pushed = False
            dist.all_reduce(self._token, group=self.pg)

    gather = finish


class StagedShardedStep(_GradIntake):
    """Sharded step cut into stages whose parameter all-gathers overlap the next stage's kernels.

    The tensors a rank owns are split into ``blocks`` groups; build the optimizer with
    :meth:`param_groups` (one param group per block - the optimizer classes run their param groups one
    after the other) and attach :meth:`after_group` as the optimizer's ``after_group`` hook.  After the
    kernels of block b are enqueued, the all-gather of block b starts on a second stream while block
    b+1 computes; :meth:`finish` joins the streams at the end of the step.
    """

    def __init__(self, shapes: Sequence[Tuple[int, ...]], device, blocks: int = 4, init_scale: float = 0.02,
                 seed: int = 1, process_group=None, cost=None):
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.blocks = blocks if self.world > 1 else 1
        shapes = [tuple(s) for s in shapes]
        self.owner, self.block, self.offsets, self.subs = partition_blocks(shapes, self.world, self.blocks, cost)
        self.base = [sum(self.subs[:b]) * self.world for b in range(self.blocks)]
        self.flat = torch.zeros(sum(self.subs) * self.world, dtype=torch.float32, device=device)
        gen = torch.Generator(device=device)
        self.params = []
        for i, (off, s) in enumerate(zip(self.offsets, shapes)):
            view = self.flat[off:off + _numel(s)].view(s)
            gen.manual_seed(seed * 1000003 + i)
            view.normal_(0.0, init_scale, generator=gen)
            self.params.append(torch.nn.Parameter(view, requires_grad=True))
        self.owned = [i for i, r in enumerate(self.owner) if r == self.rank]
        self.shard = sum(self.subs)
        self._comm = torch.cuda.Stream(device=device) if self.world > 1 and torch.device(device).type == "cuda" else None
        self._works = []

    def _grad_segments(self):
        return [(self.base[b], self.subs[b]) for b in range(self.blocks)]

    def param_groups(self, is_embedding=None):
        """Param groups in block order: one per block, or two (ordinary tensors, then embedding-like
        ones flagged ``is_embedding=True`` for the CELO2 family) when ``is_embedding(shape)`` is given."""
        out, info = [], []
        for b in range(self.blocks):
            mine = [self.params[i] for i in self.owned if self.block[i] == b]
            if is_embedding is None:
                parts = [({}, mine)]
            else:
                parts = [({}, [p for p in mine if not is_embedding(tuple(p.shape))]),
                         ({"is_embedding": True}, [p for p in mine if is_embedding(tuple(p.shape))])]
            # empty parts are dropped, but every rank keeps at least one group per block - empty if it owns nothing
            # there - because the group that closes a block starts the block's all-gather, and all ranks must start
            # the same gathers in the same order
            parts = [(extra, ps) for extra, ps in parts if ps] or [({}, [])]
            for k, (extra, ps) in enumerate(parts):
                out.append(dict(params=ps, **extra))
                info.append((b, k == len(parts) - 1))
        self._group_info = info
        return out

    def after_group(self, gi: int):
        """Hook for the optimizer: param group ``gi`` is enqueued; when it closes a block, start that
        block's all-gather."""
        if self.world == 1:
            return
        b, closes = self._group_info[gi]
        if not closes:
            return
        sub = self.subs[b]
        block = self.flat[self.base[b]:self.base[b] + self.world * sub]
        mine = block[self.rank * sub:(self.rank + 1) * sub]
        if self._comm is None:   # host tensors (the gloo tests of the layout and of the order of the gathers)
            self._works.append(dist.all_gather_into_tensor(block, mine, group=self.pg, async_op=True))
            return
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self._comm):
            self._comm.wait_event(ev)
            self._works.append(dist.all_gather_into_tensor(block, mine, group=self.pg, async_op=True))

    def finish(self):
        """Make the current stream wait for every gather of this step."""
        for w in self._works:
            w.wait()
        self._works = []

    def gather(self):
        """Non-overlapped fallback: gather every block now (used when no hook was attached)."""
        if self.world == 1:
            return
        for gi in range(len(self._group_info)):
            self.after_group(gi)
        self.finish()


def sharded_optimizer(cls, shard: ShardedStep, **kwargs):
    """Build ``cls`` over the tensors this rank owns, wired for the exchanges its family needs.

    * CELO2 / ELO_CELO2 / ELO with ``clip_grad``: the global gradient norm is the sum over ranks
      (one scalar all-reduce per step).
    * VeLO: the per-tensor LSTM inputs of all tensors are summed over ranks ([T, 30] floats) and every
      rank runs the LSTM for all T tensors; pass the same ``loss`` on every rank.
    * AdafacLO needs nothing.
    Call ``shard.gather()`` after ``optimizer.step()``.
    """
    params = [shard.params[i] for i in shard.owned]
    if cls.__name__ == "VeLO_CUDA":
        shapes = [tuple(p.shape) for p in shard.params]
        return cls(params, process_group=shard.pg, all_shapes=shapes, owned=shard.owned, **kwargs)
    opt = cls(params, **kwargs)
    if hasattr(opt, "_sharded"):
        opt._sharded = shard.world > 1
        opt.process_group = shard.pg
    return opt


def consolidate_state_dict(optimizer, shard, dst: int = 0):
    """The single-process ``state_dict`` of a sharded run, rebuilt on rank ``dst`` (``None`` elsewhere).

    Every rank's optimizer holds the state of the tensors it owns.  This gathers them (as CPU tensors)
    and re-keys them by the tensor's position in the global parameter order, which is exactly what an
    optimizer built over *all* parameters in one process would save, so the result loads into such an
    optimizer (or into the reference's classes).  Param-group hyper-parameters are taken from this
    rank's first group.  VeLO's extra entries (``loss_buffer``, ``lstm_hidden_state``, ``num_steps``) are
    replicated on every rank and are copied from rank ``dst``.
    """
    local = optimizer.state_dict()
    order = [i for g in optimizer.param_groups for i in _global_indices(g["params"], shard)]
    to_cpu = lambda v: v.detach().cpu() if torch.is_tensor(v) else v
    mine = {order[k]: {name: to_cpu(v) for name, v in st.items()} for k, st in local["state"].items()}
    world = shard.world
    gathered = [None] * world if (shard.rank == dst or world == 1) else None
    if world > 1:
        dist.gather_object(mine, gathered, dst=dst, group=shard.pg)
    else:
        gathered = [mine]
    if shard.rank != dst:
        return None
    state = {}
    for part in gathered:
        state.update(part)
    group = {k: v for k, v in local["param_groups"][0].items() if k != "params"}
    group["params"] = list(range(len(shard.params)))
    out = {"state": {i: state[i] for i in sorted(state)}, "param_groups": [group]}
    for extra in ("loss_buffer", "lstm_hidden_state", "num_steps"):
        if extra in local:
            out[extra] = local[extra]
    return out


def _global_indices(params, shard):
    pos = {id(p): i for i, p in enumerate(shard.params)}
    return [pos[id(p)] for p in params]
