"""The C-ABI library loads and exports every symbol that include/pylo_b200.h declares (no GPU needed)."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pylo_b200.h")).read()
    return sorted(set(re.findall(r"^\s*(?:int|int64_t)\s+(pylo_b200_\w+)\s*\(", text, flags=re.M)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("pylo_b200_rowcol_sums", "pylo_b200_factor_update", "pylo_b200_state_moments",
                 "pylo_b200_finalize_moments", "pylo_b200_prep_apply", "pylo_b200_apply", "pylo_b200_adamw",
                 "pylo_b200_celo2_post_sums", "pylo_b200_celo2_post_apply", "pylo_b200_grad_sumsq",
                 "pylo_b200_velo_rnn", "pylo_b200_velo_tensor_features", "pylo_b200_velo_loss_features"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from pylo_b200 import build

    path = build.build()  # nvcc cross-compiles without a GPU; a prebuilt library is reused
    lib = ctypes.CDLL(path)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_layouts_match_the_library():
    from pylo_b200 import _lib as L

    assert L.lib.pylo_b200_abi_version() == L.ABI_VERSION
    assert L.lib.pylo_b200_sizeof_desc() == L.DESC_DTYPE.itemsize
    assert L.lib.pylo_b200_sizeof_params() == ctypes.sizeof(L.StepParams)
    assert set(declared_symbols()) <= set(L.EXPORTED), "the ctypes binding must cover the whole header"


def test_argument_errors_are_reported_not_raised():
    from pylo_b200 import _lib as L

    # null descriptor table: rejected on the host with a negative code, nothing is launched
    assert L.lib.pylo_b200_finalize_moments(None, 1, None) < 0
    assert L.lib.pylo_b200_apply(None, None, 1, 0, None, None) < 0


def test_workspace_layout_is_host_only_and_consistent():
    """pylo_b200_workspace_layout / _bytes launch nothing, so they can be checked without a GPU: sizes follow the
    descriptor comments in the header, every sub-buffer is padded to 256 bytes, bad geometry is refused."""
    import ctypes as C

    from pylo_b200 import _lib as L

    w = L.workspace_layout(L.FAM_ADAFAC, L.MODE_FAST2D, 4096 * 4096, 4096, 4096, 4096, 4096)
    assert (w.f_a, w.f_b, w.sum_a, w.sum_b, w.fx) == (3 * 4096, 3 * 4096, 4096, 4096, 4 * 4096)
    assert (w.rb, w.n_strips, w.n_cb) == (32, 128, 4) and w.part_a == 4096 * 4 and w.part_b == 128 * 4096
    assert w.h_a == 4096 * 32 * 2 and w.h_b == 4096 * 32
    assert w.n_tiles == 4096 * 4096 // L.TILE_ELEMS and w.tile_part == w.n_tiles * L.STAT_STRIDE
    assert (w.closed, w.sums, w.wfold) == (L.STAT_STRIDE, L.SUMS_STRIDE, L.WFOLD_STRIDE)
    both = L.lib.pylo_b200_workspace_bytes(C.byref(w), 1, 1)
    assert both == L.lib.pylo_b200_workspace_bytes(C.byref(w), 1, 0) + L.lib.pylo_b200_workspace_bytes(C.byref(w), 0, 1)
    assert both % 256 == 0 and both >= 4 * (w.part_b + w.tile_part)
    v = L.workspace_layout(L.FAM_VELO, L.MODE_VEC1D, 1000)
    assert (v.f_a, v.h_a, v.part_b, v.n_tiles) == (0, 0, 0, 1)
    g = L.workspace_layout(L.FAM_CELO2, L.MODE_GENERIC, 768 * 3 * 16 * 16, 768 * 3 * 16, 768 * 16)
    assert (g.f_a, g.f_b, g.fx, g.h_a) == (3 * 768 * 48, 3 * 768 * 16, 0, 0)
    out = L.WsLayout()
    assert L.lib.pylo_b200_workspace_layout(L.FAM_ADAFAC, L.MODE_FAST2D, 30, 5, 6, 5, 6, C.byref(out)) == -1  # Y % 4 != 0
    assert L.lib.pylo_b200_workspace_layout(7, L.MODE_VEC1D, 30, 0, 0, 0, 0, C.byref(out)) == -1
