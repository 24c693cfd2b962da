"""Host-side logic that needs no GPU: factored-dims rules, geometry, tiling, ownership, flat layout."""

import numpy as np
import pytest
import torch

from oracle import pylo_oracle as O
from pylo_b200 import _lib as L
from pylo_b200 import plan, workloads, zero
from pylo_b200.optim import _common as K

SHAPES = [(64, 32), (32, 64), (48, 48), (7, 5, 3), (12, 3, 4, 4), (4, 4, 9, 9), (768, 3, 16, 16), (5,), ()]


@pytest.mark.parametrize("shape", SHAPES)
def test_factored_dims_rules_agree_with_the_oracle(shape):
    assert K.factored_dims_sorted(shape) == O.factored_dims_sorted(shape)
    assert K.factored_dims_argsort(shape) == O.factored_dims_argsort(shape)
    assert K.factored_dims_velo(shape) == O.factored_dims_velo(shape)


def test_velo_tie_rule():
    assert K.factored_dims_velo((1024, 1024)) == (1, 0)       # equal sizes swap (velo_cuda.py:121-131)
    assert K.factored_dims_velo((8, 8, 3, 3)) == (0, 1)       # except 4-D with axes (0, 1)
    assert K.factored_dims_sorted((4096, 4096)) == (0, 1)


@pytest.mark.parametrize("shape", [s for s in SHAPES if len(s) >= 2])
def test_geometry_indexes_like_broadcasting(shape):
    """a / b vector indices from the 5-D view equal what broadcasting a keep-dim vector would read."""
    fd = K.factored_dims_argsort(shape)
    dc, dr = fd
    Ov, X, M, Y, I, r_is_a = plan.geometry(shape, fd)
    n = int(np.prod(shape))
    idx = np.arange(n)
    i = idx % I; t = idx // I; y = t % Y; t //= Y; m = t % M; t //= M; x = t % X; o = t // X
    a = ((o * X + x) * M + m) * I + i
    b = ((o * M + m) * Y + y) * I + i
    r_shape, c_shape = list(shape), list(shape)
    r_shape[dr], c_shape[dc] = 1, 1
    rvec = np.arange(int(np.prod(r_shape))).reshape(r_shape)
    cvec = np.arange(int(np.prod(c_shape))).reshape(c_shape)
    r_b = np.broadcast_to(rvec, shape).reshape(-1)
    c_b = np.broadcast_to(cvec, shape).reshape(-1)
    assert np.array_equal(r_b, a if r_is_a else b)
    assert np.array_equal(c_b, b if r_is_a else a)


def test_tiles_cover_every_element_once():
    sizes = [1, L.TILE_ELEMS, L.TILE_ELEMS + 1, 5 * L.TILE_ELEMS - 3]
    tiles, ranges = plan.make_tiles(sizes)
    for i, n in enumerate(sizes):
        t0, k = ranges[i]
        mine = tiles[t0:t0 + k]
        assert (mine["tensor"] == i).all()
        assert mine["start"][0] == 0 and (np.diff(mine["start"]) == L.TILE_ELEMS).all()
        assert mine["start"][-1] < n <= mine["start"][-1] + L.TILE_ELEMS


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_is_deterministic_balanced_and_total(world):
    shapes = workloads.llama3_8b()
    owner = zero.partition(shapes, world)
    assert owner == zero.partition(shapes, world)
    loads = [sum(workloads.numel(s) for s, o in zip(shapes, owner) if o == r) for r in range(world)]
    assert sum(loads) == workloads.total_params(shapes)
    assert max(loads) / (sum(loads) / world) < 1.01
    offsets, shard = zero.flat_layout(shapes, owner, world)
    spans = sorted((off, off + workloads.numel(s)) for off, s in zip(offsets, shapes))
    assert all(a1 <= b0 for (_, a1), (b0, _) in zip(spans, spans[1:])), "tensors overlap in the flat buffer"
    assert all(off % zero.ALIGN == 0 for off in offsets)
    assert all(o * shard <= off < (o + 1) * shard for off, o in zip(offsets, owner))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("wl", ["llama3_8b", "gpt2_medium"])
def test_block_layout_keeps_gather_ranges_contiguous_and_tight(world, wl):
    shapes = workloads.WORKLOADS[wl]()
    blocks = 4
    owner, block, offsets, subs = zero.partition_blocks(shapes, world, blocks)
    total = workloads.total_params(shapes)
    spans = sorted((off, off + workloads.numel(s)) for off, s in zip(offsets, shapes))
    assert all(a1 <= b0 for (_, a1), (b0, _) in zip(spans, spans[1:])), "tensors overlap"
    base = [sum(subs[:b]) * world for b in range(blocks)]
    for off, s, o, b in zip(offsets, shapes, owner, block):
        lo = base[b] + o * subs[b]
        assert lo <= off and off + workloads.numel(s) <= lo + subs[b], "tensor outside its (block, rank) cell"
    if wl == "llama3_8b":
        assert sum(subs) * world < 1.01 * total  # indivisible 525 M-element tensors must not inflate the buffer


def test_workload_sizes():
    assert workloads.total_params(workloads.mlp_784()) == 118282
    assert workloads.total_params(workloads.celo2_4096()) == 4096 * 4096 + 4096
    assert abs(workloads.total_params(workloads.llama3_8b()) - 8.03e9) < 1e7
    assert abs(workloads.total_params(workloads.gpt2_medium()) - 354.8e6) < 1e6
    assert abs(workloads.total_params(workloads.vit_b16()) - 86.6e6) < 1e6


def test_cuda_classes_refuse_to_run_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from pylo_b200 import models, optim

    p = [torch.nn.Parameter(torch.zeros(4, 4))]
    with pytest.raises(RuntimeError):
        optim.CELO2_CUDA(p, network=models.CELO2MLP())
    with pytest.raises(RuntimeError):
        optim.AdafacLO_CUDA(p, network=models.MetaMLP(39, 32, 1))


@pytest.mark.parametrize("tc", [False, True])
@pytest.mark.parametrize("family", [L.FAM_ADAFAC, L.FAM_CELO2])
@pytest.mark.parametrize("X,Y", [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096), (40, 4100), (129, 300), (64, 128)])
def test_apply_items_cover_a_tensor_exactly_once(family, X, Y, tc):
    """Work items of the tiled apply sweeps: whole rows x column blocks, every element in exactly one item."""
    if tc and family != L.FAM_ADAFAC:
        pytest.skip("tensor-core kernels exist for the AdafacLO family only")
    rt, width, tag = plan.apply_tile_shape(family, X, Y, tc)
    n_r, n_c = (X + rt - 1) // rt, (Y + width - 1) // width
    assert (n_r - 1) * rt < X <= n_r * rt and (n_c - 1) * width < Y <= n_c * width
    if tc:
        assert width == 128 and tag == rt and rt in (8, 16, 32, 64)
        # as many rows per item as leave every warpgroup at least eight items, never below eight rows
        workers = L.TC_WORKERS
        assert rt == 8 or n_r * n_c >= 8 * workers
        if rt < 64:
            assert ((X + 2 * rt - 1) // (2 * rt)) * n_c < 8 * workers
    elif family == L.FAM_ADAFAC:
        assert width in (32, 64, 128, 256) and tag & 0xffff == width and rt == 32 * (tag >> 16)
    else:
        assert width == 4 * tag and rt == 16 * (256 // tag)


def test_mulo_groups_follow_the_infinite_width_shapes():
    """MuLO_cuda.py:32-60: matrix-like parameters are grouped by width multiplier with lr / width_mult, the others
    keep lr; checked on stand-ins for mup's ``infshape`` (the grouping needs nothing else of mup)."""
    from pylo_b200.optim.MuLO_cuda import mulo_param_groups

    class Inf:
        def __init__(self, n, w):
            self.n, self.w = n, w

        def ninf(self):
            return self.n

        def width_mult(self):
            return self.w

    def param(shape, n, w):
        p = torch.nn.Parameter(torch.zeros(shape))
        p.infshape = Inf(n, w)
        return p

    a, b, c, d = param((8, 8), 2, 4.0), param((8, 4), 2, 2.0), param((8,), 1, 1.0), param((4, 8), 2, 4.0)
    groups = mulo_param_groups([a, b, c, d], lr=0.5, weight_decay=0.1)
    by_lr = {g["lr"]: g["params"] for g in groups}
    assert set(by_lr) == {0.125, 0.25, 0.5}
    assert by_lr[0.125] == [a, d] and by_lr[0.25] == [b] and by_lr[0.5] == [c]
    assert all(g["weight_decay"] == 0.1 for g in groups)
    two = mulo_param_groups([{"params": [a], "lr": 1.0}, {"params": [c]}], lr=0.5)
    assert [g["lr"] for g in two if g["params"]] == [0.25, 0.5]
    with pytest.raises(AssertionError):
        mulo_param_groups([torch.nn.Parameter(torch.zeros(2, 2))])
    with pytest.raises(NotImplementedError):
        mulo_param_groups([param((2, 2, 2), 3, 1.0)])


def test_a_rank_without_tensors_still_gets_a_param_group():
    """The sharded drivers hang collectives on the optimizer's per-group hook; a rank that owns nothing must keep
    (empty) groups so that the hook still runs there."""
    from pylo_b200.zero import split_in_groups

    assert split_in_groups([], 4) == [{"params": []}]
    ps = [torch.zeros(4), torch.zeros(8), torch.zeros(4)]
    groups = split_in_groups(ps, 2)
    assert [len(g["params"]) for g in groups] == [2, 1]
