"""ctypes binding of ``libpylo_b200.so`` (the C ABI declared in include/pylo_b200.h).

There is no fallback: if the library cannot be loaded the import raises, and
every optimizer class in this package needs it.
"""

import ctypes as C
import os

import numpy as np

from . import build as _build

STAT_STRIDE = 40
SUMS_STRIDE = 48
TILE_ELEMS = 16384
A_COLS = 1024
WFOLD_STRIDE = 2432
ABI_VERSION = 10

FAM_ADAFAC, FAM_CELO2, FAM_VELO = 0, 1, 2
MODE_FAST2D, MODE_GENERIC, MODE_VEC1D = 0, 1, 2

_PTR_FIELDS = [
    "g", "p", "m", "v", "fac_a", "fac_b", "f_a", "f_b", "fx", "sum_a", "sum_b", "part_a", "part_b",
    "h_a", "h_b", "closed", "sums", "wfold", "tile_part", "out", "w", "lr_mult",
]
MAX_PEERS = 7
DESC_DTYPE = np.dtype(
    [(name, np.uint64) for name in _PTR_FIELDS]
    + [("p_peer", np.uint64, (MAX_PEERS,))]
    + [(name, np.int64) for name in ("n", "m_stride", "idx0", "La", "Lb")]
    + [(name, np.int32) for name in (
        "O", "X", "M", "Y", "I", "mode", "r_is_a", "rcm_pre", "rcm_A", "rcm_post", "rb", "n_strips", "n_cb",
        "tile0", "n_tiles", "vec_elementwise")]
    + [(name, np.float32) for name in ("lr", "wd", "step", "clip_norm", "exp_mult", "step_mult")]
    + [("n_peer", np.int32), ("pad_", np.int32)]
)
TILE_DTYPE = np.dtype([("start", np.int64), ("tensor", np.int32), ("pad_", np.int32)])
ATILE_DTYPE = np.dtype([("tensor", np.int32), ("strip", np.int32), ("cb", np.int32), ("pad_", np.int32)])
GVEC_DTYPE = np.dtype([("g", np.uint64), ("n", np.int64)])
POST_DTYPE = np.dtype(
    [("step", np.uint64), ("p", np.uint64), ("part", np.uint64), ("n", np.int64), ("tile0", np.int32),
     ("n_tiles", np.int32), ("lr", np.float32), ("wd", np.float32), ("rmsmult", np.float32), ("pad_", np.float32)]
)
ADAM_DTYPE = np.dtype(
    [("g", np.uint64), ("p", np.uint64), ("m", np.uint64), ("v", np.uint64), ("n", np.int64),
     ("lr", np.float32), ("wd", np.float32), ("bc1", np.float32), ("bc2", np.float32),
     ("clip_norm", np.float32), ("pad_", np.float32, (3,))]
)


class StepParams(C.Structure):
    _fields_ = [
        ("family", C.c_int32), ("nan_to_num", C.c_int32), ("wd_mode", C.c_int32), ("step_delta", C.c_float),
        ("w_m", C.c_float * 3), ("w_v", C.c_float), ("w_f", C.c_float * 3),
        ("eps_v", C.c_float), ("eps_feat", C.c_float), ("eps_norm", C.c_float), ("clip_val", C.c_float),
        ("no_tables", C.c_int32), ("gnorm_sq", C.c_void_p),
    ]


class WsLayout(C.Structure):
    """pylo_ws_layout: sizes in floats of a tensor's workspace sub-buffers and its phase-A / element-wise tiling."""
    _fields_ = [(name, C.c_int64) for name in (
        "f_a", "f_b", "sum_a", "sum_b", "fx", "part_a", "part_b", "h_a", "h_b", "closed", "sums", "wfold", "tile_part")] + [
        (name, C.c_int32) for name in ("rb", "n_strips", "n_cb", "n_tiles")]


class GemmDesc(C.Structure):
    """pylo_gemm_desc: C[b] = alpha * A[b] @ B[b]^T + beta * D[b] with both operands K-major."""
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("D", C.c_void_p),
                ("strideA", C.c_int64), ("strideB", C.c_int64), ("strideC", C.c_int64), ("strideD", C.c_int64)] + [
        (name, C.c_int32) for name in ("M", "N", "K", "lda", "ldb", "ldc", "ldd", "batch")] + [
        ("alpha", C.c_float), ("beta", C.c_float), ("symmetric", C.c_int32), ("pad_", C.c_int32)]


class VeloRnn(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in (
        "mix2_w", "mix2_b", "fmix_w", "fmix_b", "lstm_w", "lstm_b", "ctrl_w", "ctrl_b", "step_w", "step_b",
        "bank", "h", "c", "x_in", "pooled", "xmix", "gates", "controls", "weights", "lr_mult")] + [
        ("T", C.c_int32), ("H", C.c_int32), ("B", C.c_int32), ("pad_", C.c_int32)]


class PyloLibError(RuntimeError):
    pass


def _load():
    path = _build.LIB_PATH
    if _build.is_stale() and _build.find_nvcc() is not None:
        _build.build()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing and nvcc is not available to build it; "
            "run `python -m pylo_b200.build` where the CUDA toolkit is installed"
        )
    lib = C.CDLL(path)
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    sigs = {
        "pylo_b200_abi_version": [],
        "pylo_b200_sizeof_desc": [],
        "pylo_b200_sizeof_params": [],
        "pylo_b200_workspace_layout": [i32, i32, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.POINTER(WsLayout)],
        "pylo_b200_workspace_bytes": [C.POINTER(WsLayout), i32, i32],
        "pylo_b200_grad_sumsq": [vp, vp, i32, vp, vp, vp],
        "pylo_b200_grad_sumsq_static": [vp, vp, i32, vp, vp],
        "pylo_b200_rowcol_sums": [vp, vp, i32, vp, i32, vp, i32, C.POINTER(StepParams), vp],
        "pylo_b200_factor_update": [vp, i32, C.POINTER(StepParams), vp],
        "pylo_b200_state_moments": [vp, vp, i32, i32, C.POINTER(StepParams), vp],
        "pylo_b200_finalize_moments": [vp, i32, vp],
        "pylo_b200_prep_apply": [vp, i32, C.POINTER(StepParams), vp],
        "pylo_b200_apply": [vp, vp, i32, i32, C.POINTER(StepParams), vp],
        "pylo_b200_apply_adafac_cols": [vp, vp, i32, C.POINTER(StepParams), vp],
        "pylo_b200_apply_adafac_tc": [vp, vp, i32, C.POINTER(StepParams), vp, vp],
        "pylo_b200_apply_packed": [vp, vp, i32, C.POINTER(StepParams), vp],
        "pylo_b200_gemm_tn_3xtf32": [C.POINTER(GemmDesc), vp, vp],
        "pylo_b200_transpose": [vp, vp, i32, i32, i32, i32, C.c_int64, C.c_int64, i32, i32, vp],
        "pylo_b200_celo2_post_sums": [vp, vp, i32, vp],
        "pylo_b200_celo2_post_apply": [vp, vp, i32, vp],
        "pylo_b200_adamw": [vp, vp, i32, i32, f32, f32, f32, f32, f32, C.POINTER(StepParams), vp],
        "pylo_b200_velo_tensor_features": [vp, i32, vp, i32, vp, vp, vp, vp, vp],
        "pylo_b200_velo_rnn": [C.POINTER(VeloRnn), vp],
        "pylo_b200_velo_loss_features": [vp, vp, vp, vp, vp, vp, vp],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is missing
        fn.argtypes = argtypes
        fn.restype = C.c_int64 if name == "pylo_b200_workspace_bytes" else C.c_int
    if lib.pylo_b200_abi_version() != ABI_VERSION:
        raise ImportError("libpylo_b200.so was built from a different ABI version; rebuild it")
    if lib.pylo_b200_sizeof_desc() != DESC_DTYPE.itemsize or lib.pylo_b200_sizeof_params() != C.sizeof(StepParams):
        raise ImportError("descriptor layout mismatch between the Python binding and libpylo_b200.so")
    return lib, sorted(sigs)


lib, EXPORTED = _load()


TC_WORKERS = 148 * 4  # warpgroups the tensor-core apply kernel runs at once (four per SM)
STATIC_SCRATCH_TILES = 65536
ERR_STATIC_SCRATCH_TOO_SMALL = -4


def workspace_layout(family, mode, n, La=0, Lb=0, X=0, Y=0) -> WsLayout:
    """``pylo_b200_workspace_layout`` for one tensor (or one slice unit); raises if the library rejects the geometry."""
    out = WsLayout()
    check(lib.pylo_b200_workspace_layout(family, mode, n, La, Lb, X, Y, C.byref(out)), "workspace_layout")
    return out


def check(code, what):
    """Turn a non-zero return code of the C ABI into an exception."""
    if code == ERR_STATIC_SCRATCH_TOO_SMALL:
        raise PyloLibError(f"{what}: more than {STATIC_SCRATCH_TILES} tiles ({STATIC_SCRATCH_TILES * TILE_ELEMS} "
                           "elements) do not fit the library's built-in scratch array; pass a scratch buffer instead")
    if code != 0:
        kind = "argument rejected" if code < 0 else "CUDA error"
        raise PyloLibError(f"{what}: {kind} (code {code})")
