"""The C-ABI library loads and exports every symbol that include/pylo_b200.h declares (no GPU needed)."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pylo_b200.h")).read()
    return sorted(set(re.findall(r"^\s*int\s+(pylo_b200_\w+)\s*\(", text, flags=re.M)))


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
