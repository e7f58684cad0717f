"""Swap the reference's triangle-multiplication modules for their B200 twins at run time.

The reference picks a backend through ``ImplementationType`` in the module constructors
(``src/miniworld_engine/modules/triangle_multiplication/module.py:94-131``); a patched checkout
adds a member for this backend (the patch ships under ``integration/``).  Where the reference cannot be patched,
``install`` does the equivalent on a model that has already been built: every
``TriangleMultiplication`` / ``BidirectionalTriangleMultiplication`` submodule is replaced by
``TriangleMultiplicationB200`` / ``BidirectionalTriangleMultiplicationB200`` holding the same
parameters (same ``state_dict`` keys, device and dtype).  Modules are recognised by class name and
by the parameters they own, so the reference package itself is not imported here.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .bidirectional import BidirectionalTriangleMultiplicationB200
from .module import TriangleMultiplicationB200

__all__ = ["from_reference", "install"]

_PARAMS = ("ln_pair", "to_left", "to_left_gate", "to_right", "to_right_gate", "ln_out", "to_gate", "to_out")
_UNIDIRECTIONAL = ("TriangleMultiplication", "TriangleMultiplicationReference")
_BIDIRECTIONAL = ("BidirectionalTriangleMultiplication",)


def _looks_like_trimul(m: nn.Module) -> bool:
    return all(hasattr(m, n) and hasattr(getattr(m, n), "weight") for n in _PARAMS)


@torch.no_grad()
def from_reference(m: nn.Module) -> nn.Module:
    """The B200 twin of one reference module instance (parameters copied, same device/dtype/mode)."""
    name = type(m).__name__
    if not _looks_like_trimul(m):
        raise TypeError(f"{name} does not have the parameters of a triangle-multiplication module")
    d_pair = int(m.to_gate.weight.shape[0])
    wide = int(m.to_left.weight.shape[0])
    p_drop = float(getattr(m, "p_drop", 0.0) or 0.0)
    bidirectional = name in _BIDIRECTIONAL or (name not in _UNIDIRECTIONAL and wide == 2 * d_pair)
    if bidirectional:
        if wide % 2 or int(m.to_out.weight.shape[1]) != wide:
            raise TypeError(f"{name}: projections of width {wide} do not match to_out {tuple(m.to_out.weight.shape)}")
        twin = BidirectionalTriangleMultiplicationB200(d_pair, wide // 2, p_drop=p_drop)
    elif wide == d_pair:
        if not hasattr(m, "outgoing"):
            raise TypeError(f"{name} has no `outgoing` attribute")
        twin = TriangleMultiplicationB200(d_pair, outgoing=bool(m.outgoing), p_drop=p_drop)
    else:
        raise TypeError(f"cannot tell which block {name} is (projection width {wide}, d_pair {d_pair})")
    for attr in ("ln_pair", "ln_out"):
        eps = getattr(getattr(m, attr), "eps", None)
        if eps is not None:
            getattr(twin, attr).eps = float(eps)
    twin.load_state_dict({k: v for k, v in m.state_dict().items() if k.split(".")[0] in _PARAMS})
    ref_w = m.to_left.weight
    twin = twin.to(device=ref_w.device, dtype=ref_w.dtype)
    twin.train(m.training)
    return twin


def install(model: nn.Module) -> int:
    """Replace, in place, every reference triangle-multiplication submodule of ``model`` by its
    B200 twin.  Returns the number of modules replaced.  ``model`` itself is not replaced: convert
    a bare block with ``from_reference``."""
    n = 0
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            if type(child).__name__ in _UNIDIRECTIONAL + _BIDIRECTIONAL and _looks_like_trimul(child):
                setattr(parent, child_name, from_reference(child))
                n += 1
    return n
