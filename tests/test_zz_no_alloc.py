"""The allocation-free gradient sum of squares against the ordinary entry point.

This file is named so that pytest collects it last: if it fails, a run that stops
at the first failure has already run everything else.

`pylo_b200_grad_sumsq_static` exists for hosts that cannot give the library a
scratch buffer (a foreign-language binding with no device allocator, or a step
loop in which cudaMalloc is off limits because it stalls the device).  It keeps
its partial sums in an array built into the library.  The checks: it returns
what `pylo_b200_grad_sumsq` returns for the same gradients, twice in a row with
different gradients (the built-in array still holds the first call's partials
when the second one starts), and it refuses more tiles than the array holds.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [5, 16384, 16385, 300_001, 4096 * 1024]


def _tables(grads, device):
    from pylo_b200 import _lib as L
    from pylo_b200 import plan

    items = np.zeros(len(grads), dtype=L.GVEC_DTYPE)
    items["n"] = [g.numel() for g in grads]
    items["g"] = [g.data_ptr() for g in grads]
    tiles, _ = plan.make_tiles([g.numel() for g in grads])
    return plan.DeviceTable(items, device), plan.DeviceTable(tiles, device), len(tiles)


def _both(grads, device):
    from pylo_b200 import _lib as L

    stream = torch.cuda.current_stream().cuda_stream
    items, tiles, n_tiles = _tables(grads, device)
    scratch = torch.zeros(n_tiles, dtype=torch.float32, device=device)
    ref = torch.zeros(1, dtype=torch.float32, device=device)
    got = torch.full((1,), -1.0, dtype=torch.float32, device=device)
    L.check(L.lib.pylo_b200_grad_sumsq(items.ptr, tiles.ptr, n_tiles, scratch.data_ptr(), ref.data_ptr(), stream), "grad_sumsq")
    L.check(L.lib.pylo_b200_grad_sumsq_static(items.ptr, tiles.ptr, n_tiles, got.data_ptr(), stream), "grad_sumsq_static")
    torch.cuda.synchronize()
    return float(ref.item()), float(got.item())


def test_static_scratch_variant_matches_twice_in_a_row():
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(11)
    first = [torch.randn(n, generator=gen, device=dev) * 3.0 for n in SIZES]
    ref1, got1 = _both(first, dev)
    exact1 = float(sum(g.double().pow(2).sum() for g in first))
    assert got1 == pytest.approx(ref1, rel=1e-6)
    assert got1 == pytest.approx(exact1, rel=1e-5)
    # second call: fewer, smaller, differently scaled gradients, so stale partials would show
    second = [torch.randn(n, generator=gen, device=dev) * 0.01 for n in SIZES[:3]]
    ref2, got2 = _both(second, dev)
    exact2 = float(sum(g.double().pow(2).sum() for g in second))
    assert got2 == pytest.approx(ref2, rel=1e-6)
    assert got2 == pytest.approx(exact2, rel=1e-5)
    assert got2 < got1 * 1e-3


def test_static_scratch_variant_refuses_what_does_not_fit():
    from pylo_b200 import _lib as L

    dev = torch.device("cuda", 0)
    g = torch.ones(8, device=dev)
    items, tiles, _ = _tables([g], dev)
    out = torch.zeros(1, device=dev)
    rc = L.lib.pylo_b200_grad_sumsq_static(items.ptr, tiles.ptr, L.STATIC_SCRATCH_TILES + 1, out.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == L.ERR_STATIC_SCRATCH_TOO_SMALL
    with pytest.raises(L.PyloLibError, match="built-in scratch"):
        L.check(rc, "grad_sumsq_static")


def test_static_scratch_variant_allocates_nothing():
    """After the set-up call (which looks up the built-in array's address) a call on tables that already exist
    must leave the device's free memory and torch's allocator counters exactly where they were."""
    from pylo_b200 import _lib as L

    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(12)
    grads = [torch.randn(n, generator=gen, device=dev) for n in SIZES[:4]]
    items, tiles, n_tiles = _tables(grads, dev)
    out = torch.zeros(1, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    L.check(L.lib.pylo_b200_grad_sumsq_static(items.ptr, tiles.ptr, n_tiles, out.data_ptr(), stream), "set-up call")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    alloc0, reserved0 = torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for _ in range(3):
        L.check(L.lib.pylo_b200_grad_sumsq_static(items.ptr, tiles.ptr, n_tiles, out.data_ptr(), stream), "grad_sumsq_static")
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)) == (alloc0, reserved0)
    assert free1 == free0, "the allocation-free entry point changed the device's free memory"
    assert float(out.item()) == pytest.approx(float(sum(g.double().pow(2).sum() for g in grads)), rel=1e-5)


def test_static_scratch_variant_on_a_second_device():
    """The built-in array exists once per GPU and its address is looked up per device: repeat the comparison on
    cuda:1 where there is one."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    dev = torch.device("cuda", 1)
    with torch.cuda.device(dev):
        gen = torch.Generator(device=dev).manual_seed(13)
        grads = [torch.randn(n, generator=gen, device=dev) * 2.0 for n in SIZES[:4]]
        ref, got = _both(grads, dev)
        assert got == pytest.approx(ref, rel=1e-6)
        assert got == pytest.approx(float(sum(g.double().pow(2).sum() for g in grads)), rel=1e-5)
