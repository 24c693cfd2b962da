"""Host-side planning for the multi-tensor step: descriptor tables, tile lists, workspace.

The optimizer classes describe every tensor on the learned-optimizer path with
a :class:`LoTensor`; :class:`LoPlan` turns the list into the device-resident
tables the C ABI works on (include/pylo_b200.h) and issues the fixed launch
sequence of one step.  Nothing here touches tensor values on the host.
"""

from __future__ import annotations

import contextlib
import ctypes as C
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib as L


def _prod(xs) -> int:
    out = 1
    for x in xs:
        out *= int(x)
    return out


@dataclass
class LoTensor:
    """One tensor on the learned-optimizer path (all tensors fp32, contiguous, on one CUDA device)."""

    p: torch.Tensor
    m: torch.Tensor                     # (3,) + shape
    v: torch.Tensor                     # shape or (1,) + shape
    fac_r: Optional[torch.Tensor]       # [3] + shape[dr -> 1]; fewer than 2 dims: (3,) + shape
    fac_c: Optional[torch.Tensor]       # [3] + shape[dc -> 1]; fewer than 2 dims: (3,) + shape or None
    fdims: Optional[Tuple[int, int]]    # (dc, dr) or None for fewer than 2 dims
    rcm_axis: int = 0                   # axis of fac_r over which row_col_mean is taken
    lr: float = 1e-3
    wd: float = 0.0
    clip_norm: float = 0.0
    exp_mult: float = 0.0
    step_mult: float = 1.0
    out: Optional[torch.Tensor] = None  # CELO2 raw step
    w: Optional[torch.Tensor] = None    # network weights in family layout
    lr_mult: Optional[torch.Tensor] = None
    slice_last2: bool = False           # normalise features per matrix (last two axes) instead of per tensor
    peer_ptrs: Optional[Sequence[int]] = None  # device addresses of this parameter in the other ranks' buffers
    peer_multicast: bool = False  # peer_ptrs holds ONE multicast address that maps the parameter on every rank


def geometry(shape: Sequence[int], fdims):
    """(O, X, M, Y, I, r_is_a) of a contiguous tensor whose factored axes are fdims = (dc, dr)."""
    dc, dr = fdims
    ax, ay = (dc, dr) if dc < dr else (dr, dc)
    O = _prod(shape[:ax])
    X = int(shape[ax])
    M = _prod(shape[ax + 1:ay])
    Y = int(shape[ay])
    I = _prod(shape[ay + 1:])
    return O, X, M, Y, I, int(dr == ay)


def _aligned16(*tensors) -> bool:
    return all(t is None or t.data_ptr() % 16 == 0 for t in tensors)


def make_tiles(sizes: Sequence[int]) -> Tuple[np.ndarray, List[Tuple[int, int]]]:
    """Element-wise tiles over items of the given sizes; returns (tiles, [(tile0, n_tiles)] per item)."""
    ranges, total = [], 0
    for n in sizes:
        k = (int(n) + L.TILE_ELEMS - 1) // L.TILE_ELEMS
        ranges.append((total, k))
        total += k
    tiles = np.zeros(total, dtype=L.TILE_DTYPE)
    for i, (t0, k) in enumerate(ranges):
        tiles["tensor"][t0:t0 + k] = i
        tiles["start"][t0:t0 + k] = np.arange(k, dtype=np.int64) * L.TILE_ELEMS
    return tiles, ranges


class DeviceTable:
    """A numpy structured array mirrored in device memory through two pinned staging buffers."""

    def __init__(self, host: np.ndarray, device):
        self.host = host
        self.nbytes = max(host.nbytes, 16)
        self.dev = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self._stage = [torch.empty(self.nbytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self._events = [None, None]
        self._turn = 0
        self._last = None
        self.upload()

    @property
    def ptr(self) -> int:
        return self.dev.data_ptr()

    def upload(self):
        """Copy the host array to the device unless it still holds exactly these bytes."""
        raw = self.host.view(np.uint8).reshape(-1) if self.host.nbytes else None
        if raw is not None and self._last is not None and np.array_equal(raw, self._last):
            return
        self._last = None if raw is None else raw.copy()
        i = self._turn
        self._turn ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()
        if self.host.nbytes:
            self._stage[i].numpy()[: self.host.nbytes] = self.host.view(np.uint8).reshape(-1)
        self.dev.copy_(self._stage[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev


def apply_tile_shape(family: int, X: int, Y: int, tensor_cores=None):
    """(rows per work item, columns per work item, tag for ``pylo_atile.pad_``) of a FAST2D tensor's apply sweep.

    * tensor-core kernel (AdafacLO family, ``tensor_cores`` true): an item is rt rows x 128 columns, taken by one
      warpgroup (four per SM); as many rows as possible (the column terms are loaded once per item) while the
      tensor still yields >= 8 items per warpgroup; tag = rt;
    * AdafacLO family on the CUDA cores: n_sub sub-tiles of 32 rows in one block of 32..256 columns, as long as
      possible while the tensor still yields >= 8 items per SM; tag = columns | n_sub << 16;
    * CELO2 / VeLO: four columns per thread, tag = threads per row.
    """
    if tensor_cores:
        ncol = (Y + 127) // 128
        rt = next((r for r in (64, 32, 16) if ((X + r - 1) // r) * ncol >= 8 * L.TC_WORKERS), 8)
        return rt, 128, rt
    if family == L.FAM_ADAFAC:
        cw = min((256, 128, 64, 32), key=lambda c: ((Y + c - 1) // c * c - Y, -c))
        ncol = (Y + cw - 1) // cw
        n_sub = next((k for k in (8, 4, 2) if ((X + 32 * k - 1) // (32 * k)) * ncol >= 1184), 1)
        return 32 * n_sub, cw, cw | (n_sub << 16)
    tpr = min((256, 128, 64, 32, 16, 8), key=lambda c: ((Y + 4 * c - 1) // (4 * c) * 4 * c - Y, -c))
    return 16 * (256 // tpr), 4 * tpr, tpr


class LoPlan:
    """Descriptor tables, tile lists and workspace for the tensors of one optimizer instance.

    Two tables: one descriptor per tensor (phases A and A2 work on whole tensors) and one per
    unit of element-wise work (phases B to C).  A unit is a tensor, or one matrix slice of a
    tensor flagged ``slice_last2``; when nothing is sliced the two tables are one.
    """

    H = {L.FAM_ADAFAC: 32, L.FAM_CELO2: 8, L.FAM_VELO: 4}

    def __init__(self, family: int, tensors: List[LoTensor], device, tensor_cores=False):
        self.family = family
        # whether the AdafacLO family's FAST2D tensors take the tensor-core apply kernel (TF32 operands)
        self.tensor_cores = bool(tensor_cores) and family == L.FAM_ADAFAC
        self.tensors = tensors
        self.device = torch.device(device)
        T = len(tensors)
        H = self.H[family]
        tdesc = np.zeros(T, dtype=L.DESC_DTYPE)
        ws_items = []  # (table, row, field, count)
        atiles, rtiles, generic = [], [], []
        ws_bytes = 0  # the library's own count of the workspace, checked against the layout below
        for i, t in enumerate(tensors):
            shape = tuple(t.p.shape)
            n = t.p.numel()
            if n == 0:
                raise ValueError("empty parameter tensors are not supported on the learned-optimizer path")
            for name in ("p", "m", "v", "fac_r", "fac_c", "out"):
                x = getattr(t, name)
                if x is not None and not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
                    raise ValueError(f"{name} of tensor {i} must be a contiguous fp32 CUDA tensor")
            d = tdesc[i]
            d["n"], d["m_stride"], d["idx0"] = n, n, 0
            d["lr"], d["wd"], d["clip_norm"] = t.lr, t.wd, t.clip_norm
            d["exp_mult"], d["step_mult"] = t.exp_mult, t.step_mult
            d["p"], d["m"], d["v"] = t.p.data_ptr(), t.m.data_ptr(), t.v.data_ptr()
            d["out"] = t.out.data_ptr() if t.out is not None else 0
            d["w"] = t.w.data_ptr() if t.w is not None else 0
            d["lr_mult"] = t.lr_mult.data_ptr() if t.lr_mult is not None else 0
            if t.peer_ptrs:
                if len(t.peer_ptrs) > L.MAX_PEERS:
                    raise ValueError(f"at most {L.MAX_PEERS} peers (8 GPUs of one box)")
                d["p_peer"][: len(t.peer_ptrs)] = list(t.peer_ptrs)
                d["n_peer"] = -1 if t.peer_multicast else len(t.peer_ptrs)
            if t.fdims is None:
                d["mode"] = L.MODE_VEC1D
                d["O"] = d["X"] = d["M"] = d["I"] = 1
                d["Y"] = min(n, 2**31 - 1)
                d["r_is_a"] = 1
                d["fac_a"] = t.fac_r.data_ptr()
                d["fac_b"] = t.fac_c.data_ptr() if t.fac_c is not None else 0
                d["rcm_pre"] = d["rcm_A"] = d["rcm_post"] = 1
            else:
                O, X, M, Y, I, r_is_a = geometry(shape, t.fdims)
                d["O"], d["X"], d["M"], d["Y"], d["I"], d["r_is_a"] = O, X, M, Y, I, r_is_a
                La, Lb = n // Y, n // X
                d["La"], d["Lb"] = La, Lb
                fac_a, fac_b = (t.fac_r, t.fac_c) if r_is_a else (t.fac_c, t.fac_r)
                d["fac_a"], d["fac_b"] = fac_a.data_ptr(), fac_b.data_ptr()
                rshape = list(t.fac_r.shape)
                ax = t.rcm_axis
                d["rcm_pre"], d["rcm_A"], d["rcm_post"] = _prod(rshape[:ax]), rshape[ax], _prod(rshape[ax + 1:])
                fast = (O == 1 and M == 1 and I == 1 and Y % 4 == 0 and n < 2**31
                        and not (t.slice_last2 and t.p.dim() > 2) and _aligned16(t.p, t.m, t.v, t.out))
                d["mode"] = L.MODE_FAST2D if fast else L.MODE_GENERIC
                # sub-buffer sizes and the phase-A tiling come from the library (pylo_b200_workspace_layout), so that
                # this table and a table built by any other host of the C ABI agree
                ws = L.workspace_layout(family, int(d["mode"]), n, La, Lb, X if fast else 0, Y if fast else 0)
                ws_items += [("t", i, f, getattr(ws, f)) for f in ("f_a", "f_b", "sum_a", "sum_b")]
                if fast:
                    d["rb"], d["n_strips"], d["n_cb"] = ws.rb, ws.n_strips, ws.n_cb
                    assert ws.rb == min(128, max(32, ((X + 127) // 128 + 7) // 8 * 8)) and ws.h_a == La * H * 2
                    ws_items += [("t", i, f, getattr(ws, f)) for f in ("fx", "part_a", "part_b", "h_a", "h_b")]
                    for s in range(ws.n_strips):
                        for cb in range(ws.n_cb):
                            atiles.append((i, s, cb, 0))
                    rtiles += [(i, 0, cb, 0) for cb in range(ws.n_cb)]
                else:
                    generic.append(i)
            ws_items.append(("t", i, "closed", L.STAT_STRIDE))
            ws_bytes += L.lib.pylo_b200_workspace_bytes(
                C.byref(L.workspace_layout(family, int(d["mode"]), n, int(d["La"]), int(d["Lb"]),
                                           int(d["X"]) if d["mode"] == L.MODE_FAST2D else 0,
                                           int(d["Y"]) if d["mode"] == L.MODE_FAST2D else 0)), 1, 0)

        # units of element-wise work
        self.sliced = any(t.slice_last2 and t.p.dim() > 2 for t in tensors)
        unit_owner = []  # (tensor index, element offset)
        for i, t in enumerate(tensors):
            if t.slice_last2 and t.p.dim() > 2:
                mat = t.p.shape[-1] * t.p.shape[-2]
                unit_owner += [(i, k * mat) for k in range(t.p.numel() // mat)]
            else:
                unit_owner.append((i, 0))
        U = len(unit_owner)
        if self.sliced:
            udesc = np.zeros(U, dtype=L.DESC_DTYPE)
            for u, (i, off) in enumerate(unit_owner):
                udesc[u] = tdesc[i]
                t = tensors[i]
                if t.slice_last2 and t.p.dim() > 2:
                    mat = t.p.shape[-1] * t.p.shape[-2]
                    udesc["n"][u], udesc["idx0"][u], udesc["vec_elementwise"][u] = mat, off, 1
                    for f in ("p", "m", "v", "out"):
                        if udesc[f][u]:
                            udesc[f][u] += 4 * off
                    ws_items.append(("u", u, "closed", L.STAT_STRIDE))  # stays zero: no closed forms for a slice
                    ws_bytes += (L.STAT_STRIDE + 63) // 64 * 256
        else:
            udesc = tdesc
        sizes = [int(udesc["n"][u]) for u in range(U)]
        tiles, ranges = make_tiles(sizes)
        for u, (t0, k) in enumerate(ranges):
            udesc["tile0"][u], udesc["n_tiles"][u] = t0, k
            ws = L.workspace_layout(family, L.MODE_VEC1D, sizes[u])  # the per-unit part depends on the element count only
            assert ws.n_tiles == k
            ws_items += [("u", u, f, getattr(ws, f)) for f in ("sums", "wfold", "tile_part")]
            ws_bytes += L.lib.pylo_b200_workspace_bytes(C.byref(ws), 0, 1)
        # workspace: every sub-buffer starts on a 256-byte boundary
        off = 0
        placed = []
        for table, row, fld, count in ws_items:
            placed.append((table, row, fld, off))
            off += (count + 63) // 64 * 64
        if off * 4 != ws_bytes:
            raise AssertionError(f"workspace layout ({off * 4} bytes) disagrees with pylo_b200_workspace_bytes ({ws_bytes})")
        self.workspace = torch.zeros(max(off, 64), dtype=torch.float32, device=self.device)
        base = self.workspace.data_ptr()
        for table, row, fld, o in placed:
            (tdesc if table == "t" else udesc)[fld][row] = base + 4 * o
        if self.sliced:  # units inherit their tensor's factor workspace
            for u, (i, _) in enumerate(unit_owner):
                for f in ("f_a", "f_b", "fx", "sum_a", "sum_b", "part_a", "part_b", "h_a", "h_b"):
                    udesc[f][u] = tdesc[f][i]
                if not udesc["vec_elementwise"][u]:
                    udesc["closed"][u] = tdesc["closed"][i]
        self.unit_owner = unit_owner
        self.tdesc = DeviceTable(tdesc, self.device)
        self.desc = DeviceTable(udesc, self.device) if self.sliced else self.tdesc
        self.tiles = DeviceTable(tiles, self.device)
        self.n_tiles = len(tiles)
        self.atiles = DeviceTable(np.array(atiles, dtype=np.int32).reshape(-1, 4).view(L.ATILE_DTYPE).reshape(-1), self.device)
        self.n_atiles = len(atiles)
        self.rtiles = DeviceTable(np.array(rtiles, dtype=np.int32).reshape(-1, 4).view(L.ATILE_DTYPE).reshape(-1), self.device)
        self.n_rtiles = len(rtiles)
        self.generic = DeviceTable(np.array(generic, dtype=np.int32), self.device)
        self.n_generic = len(generic)
        self.n_tensors = T
        self.n_units = U
        self.total_elems = int(sum(sizes))
        self._keepalive = []
        # FAST2D tensors take a tiled apply kernel (see apply_tile_shape); everything else the generic one
        ctiles = []
        unit_of = {i: u for u, (i, _) in enumerate(unit_owner)}  # a FAST2D tensor is never sliced: one unit
        for i in range(T):
            if tdesc["mode"][i] != L.MODE_FAST2D:
                continue
            X, Y = int(tdesc["X"][i]), int(tdesc["Y"][i])
            rt, width, tag = apply_tile_shape(family, X, Y, self.tensor_cores)
            for rtile in range((X + rt - 1) // rt):
                for ctile in range((Y + width - 1) // width):
                    ctiles.append((unit_of[i], rtile, ctile, tag))
        self.ctiles = DeviceTable(np.array(ctiles, dtype=np.int32).reshape(-1, 4).view(L.ATILE_DTYPE).reshape(-1), self.device)
        self.n_ctiles = len(ctiles)
        #: the kernel that takes the FAST2D tensors' apply sweep (also the key of its timings in phase_times())
        if self.tensor_cores:
            self.apply_kernel = "k_apply_adafac_tc"
        elif family == L.FAM_ADAFAC:
            self.apply_kernel = "k_apply_adafac_cols"
        else:
            self.apply_kernel = "k_apply_packed<CELO2>" if family == L.FAM_CELO2 else "k_apply_packed<VELO>"
        #: device flag the tensor-core kernel raises when one of its bounded waits ran out
        self.status = torch.zeros(128, dtype=torch.int32, device=self.device) if self.tensor_cores else None
        # a pinned copy of the flag follows every launch without blocking; the next launch looks at it once it landed
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory() if self.tensor_cores else None
        self._status_event = None
        fast_unit = udesc["mode"] == L.MODE_FAST2D
        slow = tiles[~fast_unit[tiles["tensor"]]] if len(tiles) else tiles
        self.tiles_slow = DeviceTable(np.ascontiguousarray(slow), self.device)
        self.n_tiles_slow = len(slow)

    # ------------------------------------------------------------------ per-step refresh
    def set_field(self, name, values):
        """Set a per-tensor field (scalar or one value per tensor) in both tables."""
        self.tdesc.host[name][:] = values
        if self.sliced:
            vals = np.broadcast_to(np.asarray(values), (self.n_tensors,))
            self.desc.host[name][:] = [vals[i] for i, _ in self.unit_owner]

    def refresh(self, grads: Sequence[torch.Tensor], steps=None):
        """Point the descriptors at this step's gradients (and step counts) and upload the tables."""
        self._keepalive = []
        ptrs = np.zeros(self.n_tensors, dtype=np.uint64)
        for i, g in enumerate(grads):
            if not (g.is_cuda and g.dtype == torch.float32 and g.is_contiguous() and g.data_ptr() % 16 == 0):
                g = g.to(torch.float32).contiguous().clone()
                self._keepalive.append(g)
            ptrs[i] = g.data_ptr()
        self.tdesc.host["g"][:] = ptrs
        self.step_delta = 0.0
        if steps is not None:
            # when every tensor advanced by the same amount since the table was last written, leave the
            # table alone and hand the kernels the difference (no upload on the step path)
            delta = np.asarray(steps, dtype=np.float64) - self.tdesc.host["step"].astype(np.float64)
            if len(delta) and np.all(delta == delta[0]) and 0 <= delta[0] < 2**20 and self.tdesc._last is not None:
                self.step_delta = float(delta[0])
            else:
                self.set_field("step", steps)
        self.tdesc.upload()
        if self.sliced:
            self.desc.host["g"][:] = [ptrs[i] + np.uint64(4 * off) for i, off in self.unit_owner]
            self.desc.upload()

    # ------------------------------------------------------------------ launch sequence
    #: the kernel that dominates each timed phase, for reports
    KERNEL_OF = {"rowcol_sums": "k_rowcol_fast", "factor_update": "k_factor_update", "state_moments": "k_state_moments",
                 "finalize_moments": "k_finalize_moments", "prep_apply": "k_prep_apply"}
    #: kernels each C-ABI call launches (for the launch count the benchmark reports)
    LAUNCHES = {"rowcol_sums": 1, "factor_update": 1, "state_moments": 1, "finalize_moments": 1, "prep_apply": 1}

    def enable_profile(self, on: bool = True):
        """Record a CUDA-event pair around every phase launch (read back with :meth:`phase_times`)."""
        self._prof = {} if on else None

    def phase_times(self):
        """{phase: [ms, ...]} of the recorded launches; call after a device synchronisation."""
        return {k: [a.elapsed_time(b) for a, b in v] for k, v in (self._prof or {}).items()}

    def _call(self, name, fn, *args):
        prof = getattr(self, "_prof", None)
        if prof is not None:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        L.check(fn(*args), name)
        self.launch_count = getattr(self, "launch_count", 0) + self.LAUNCHES.get(name, 1)
        if prof is not None:
            b.record()
            prof.setdefault(name, []).append((a, b))

    def run_front(self, prm: L.StepParams, stream: int, reverse_b: bool = True):
        """Phases A, A2, B, B2."""
        self._poll_status()  # before any state of this step is touched
        prm.step_delta = getattr(self, "step_delta", 0.0)
        pp = C.byref(prm)
        if self.n_atiles or self.n_generic:
            self._call("rowcol_sums", L.lib.pylo_b200_rowcol_sums, self.tdesc.ptr, self.atiles.ptr, self.n_atiles,
                       self.rtiles.ptr, self.n_rtiles, self.generic.ptr, self.n_generic, pp, stream)
            self.launch_count += (1 if self.n_atiles else 0) + (1 if self.n_atiles and self.n_generic else 0)
        self._call("factor_update", L.lib.pylo_b200_factor_update, self.tdesc.ptr, self.n_tensors, pp, stream)
        self._call("state_moments", L.lib.pylo_b200_state_moments, self.desc.ptr, self.tiles.ptr, self.n_tiles,
                   int(reverse_b), pp, stream)
        self._call("finalize_moments", L.lib.pylo_b200_finalize_moments, self.desc.ptr, self.n_units, stream)

    def _poll_status(self):
        """Raise if the copy of the status word that followed an earlier tensor-core launch has landed non-zero."""
        if self._status_event is not None and self._status_event.query() and int(self._status_host[0]) != 0:
            raise L.PyloLibError("apply_adafac_tc: a wait on the tensor core timed out in an earlier step; the kernel "
                                 "kept the old values of the parameters it could not finish, and launches write "
                                 "nothing until clear_status() is called")

    def run_back(self, prm: L.StepParams, stream: int, reverse_c: bool = False):
        """Phases P, C."""
        # the tensor-core kernel needs the per-row table only (2); the CUDA-core kernels need both (0)
        prm.no_tables = 2 if self.tensor_cores else 0
        pp = C.byref(prm)
        self._call("prep_apply", L.lib.pylo_b200_prep_apply, self.desc.ptr, self.n_units, pp, stream)
        if self.n_ctiles and self.tensor_cores:
            self._poll_status()
            self._call(self.apply_kernel, L.lib.pylo_b200_apply_adafac_tc, self.desc.ptr, self.ctiles.ptr, self.n_ctiles, pp, self.status.data_ptr(), stream)
            # a pinned copy of the status word follows the launch on the launch's own stream, without blocking
            ctx = (torch.cuda.stream(torch.cuda.ExternalStream(stream, device=self.device))
                   if stream != current_stream_ptr() else contextlib.nullcontext())
            with ctx:
                self._status_host.copy_(self.status[:1], non_blocking=True)
                self._status_event = torch.cuda.Event()
                self._status_event.record()
        elif self.n_ctiles:
            fn = L.lib.pylo_b200_apply_adafac_cols if self.family == L.FAM_ADAFAC else L.lib.pylo_b200_apply_packed
            self._call(self.apply_kernel, fn, self.desc.ptr, self.ctiles.ptr, self.n_ctiles, pp, stream)
        if self.n_tiles_slow:
            self._call("k_apply", L.lib.pylo_b200_apply, self.desc.ptr, self.tiles_slow.ptr, self.n_tiles_slow, int(reverse_c), pp, stream)

    def check_status(self):
        """Synchronise and raise if the tensor-core kernel reported a wait that ran out.

        The kernel keeps the old value of every parameter it could not finish, so nothing invalid was written, but
        the step is incomplete; until :meth:`clear_status` the kernel stores nothing at all.  Call this before a
        checkpoint is written."""
        if self.status is not None and int(self.status[0].item()) != 0:
            raise L.PyloLibError("apply_adafac_tc: a wait on the tensor core timed out; this step is incomplete "
                                 "(unfinished parameters kept their old values)")

    def clear_status(self):
        """Acknowledge a reported timeout: the next launches store again."""
        if self.status is not None:
            self.status.zero_()
            self._status_host.zero_()
            self._status_event = None


class GradNorm:
    """Device-side sum of squares of a list of gradients (the global-norm clip)."""

    def __init__(self, sizes: Sequence[int], device):
        self.out = torch.zeros(1, dtype=torch.float32, device=device)
        self._keepalive = []
        self.n_tiles = 0
        if len(sizes) == 0:   # a rank that owns no tensor still takes part in the all-reduce of the sum: with zero
            return
        self.items = np.zeros(len(sizes), dtype=L.GVEC_DTYPE)
        self.items["n"] = sizes
        tiles, _ = make_tiles(sizes)
        self.tiles = DeviceTable(tiles, device)
        self.n_tiles = len(tiles)
        self.table = DeviceTable(self.items, device)
        self.scratch = torch.zeros(max(self.n_tiles, 1), dtype=torch.float32, device=device)

    def run(self, grads: Sequence[torch.Tensor], stream: int):
        self._keepalive = []
        if self.n_tiles == 0:
            self.out.zero_()
            return self.out
        for i, g in enumerate(grads):
            if not (g.dtype == torch.float32 and g.is_contiguous()):
                g = g.to(torch.float32).contiguous()
                self._keepalive.append(g)
            self.items["g"][i] = g.data_ptr()
        self.table.upload()
        L.check(L.lib.pylo_b200_grad_sumsq(self.table.ptr, self.tiles.ptr, self.n_tiles, self.scratch.data_ptr(),
                                           self.out.data_ptr(), stream), "grad_sumsq")
        return self.out


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def f32(x) -> float:
    """Round a Python float to fp32 the way a torch fp32 tensor element would hold it."""
    return float(np.float32(x))


def one_minus(beta: torch.Tensor) -> List[float]:
    """``1 - beta`` evaluated in fp32, as ``1 - tensor`` does in the reference classes."""
    return [float(x) for x in (1 - beta.detach().to("cpu", torch.float32)).tolist()]


INF = math.inf
