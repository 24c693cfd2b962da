"""MuLO_CUDA: the muP wrapper around AdafacLO_CUDA (pylo/optim/MuLO_cuda.py:12-61).

The wrapper does no arithmetic of its own: it splits every param group by the
infinite-width shape that ``mup.set_base_shapes`` attached to the parameters
(``p.infshape``) - matrix-like parameters (two infinite dimensions) go into one
group per width multiplier with ``lr`` divided by that multiplier, everything
else into one group that keeps ``lr`` - and builds the optimizer over the new
groups.  The step then runs on the same kernels as AdafacLO_CUDA; each group
carries its own ``lr`` into the tensor descriptors.

``mup.optim.process_param_groups`` (what the reference calls first) only
normalises the argument into a list of group dicts and fills in ``lr`` and
``weight_decay`` from the keyword arguments where a group has none.  When the
``mup`` package is installed its function is used; when it is not, the same
normalisation is done here, so the wrapper can be used (and tested) with any
objects that carry an ``infshape`` with ``ninf()`` and ``width_mult()``.
"""

from __future__ import annotations

from collections import defaultdict

from .AdafacLO_cuda import AdafacLO_CUDA


def _process_param_groups(params, **kwargs):
    try:
        from mup.optim import process_param_groups
    except ImportError:
        process_param_groups = None
    if process_param_groups is not None:
        return process_param_groups(params, **kwargs)
    groups = list(params)
    if not groups or not isinstance(groups[0], dict):
        groups = [{"params": groups}]
    out = []
    for g in groups:
        g = dict(g)
        g["params"] = list(g["params"])
        g.setdefault("lr", kwargs.get("lr", 1.0))   # AdafacLO_CUDA's default learning rate (AdafacLO_cuda.py:84)
        g.setdefault("weight_decay", kwargs.get("weight_decay", 0.0))
        out.append(g)
    return out


def mulo_param_groups(params, **kwargs):
    """The param groups MuLO builds (MuLO_cuda.py:32-60): per incoming group, one group per width multiplier for the
    matrix-like parameters (``lr / width_mult``), then one group for the vector-like ones."""
    new_groups = []
    for group in _process_param_groups(params, **kwargs):
        def new_group():
            g = {k: v for k, v in group.items() if k != "params"}
            g["params"] = []
            return g

        matrix_like = defaultdict(new_group)  # keyed by width multiplier
        vector_like = new_group()
        for p in group["params"]:
            if not hasattr(p, "infshape"):
                raise AssertionError(f"A parameter with shape {tuple(p.shape)} does not have `infshape` attribute. "
                                     "Did you forget to call `mup.set_base_shapes` on the model?")
            n_inf = p.infshape.ninf()
            if n_inf == 2:
                matrix_like[p.infshape.width_mult()]["params"].append(p)
            elif n_inf > 2:
                raise NotImplementedError("more than 2 inf dimensions")
            else:
                vector_like["params"].append(p)
        for width_mult, g in matrix_like.items():
            g["lr"] /= width_mult
        new_groups.extend(list(matrix_like.values()) + [vector_like])
    return new_groups


def MuLO_CUDA(params, impl=AdafacLO_CUDA, **kwargs):
    """muP-parameterised AdafacLO on the B200 kernels; same call signature as the reference's ``MuLO_CUDA``."""
    return impl(mulo_param_groups(params, **kwargs), **kwargs)
