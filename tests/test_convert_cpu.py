"""Run-time replacement of the reference's modules by their B200 twins (no GPU needed: only the
parameter plumbing is checked here; the numerics of the twins are covered by the GPU tests)."""

import os
import sys

import pytest
import torch
import torch.nn as nn

from miniworld_engine_b200 import (BidirectionalTriangleMultiplicationB200, TriangleMultiplicationB200,
                                   from_reference, install)



def _reference_src() -> str:
    """``src`` directory of the reference project where this machine has one: the environment
    variable MINIWORLD_REFERENCE, else the ``reference_path`` recorded in BASELINE.json."""
    root = os.environ.get("MINIWORLD_REFERENCE")
    if not root:
        try:
            import json
            with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "BASELINE.json")) as f:
                root = json.load(f).get("reference_path", "")
        except (OSError, ValueError):
            root = ""
    return os.path.join(root, "src") if root else ""


REFERENCE = _reference_src()


class _LN(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight, self.bias, self.eps = nn.Parameter(torch.randn(d)), nn.Parameter(torch.randn(d)), eps


class TriangleMultiplication(nn.Module):          # stand-in with the reference module's attribute names
    def __init__(self, d, outgoing):
        super().__init__()
        self.outgoing, self.p_drop = outgoing, 0.25
        self.ln_pair, self.ln_out = _LN(d, 1e-6), _LN(d)
        for n in ("to_left", "to_left_gate", "to_right", "to_right_gate", "to_gate", "to_out"):
            setattr(self, n, nn.Linear(d, d, bias=False))


class BidirectionalTriangleMultiplication(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.p_drop = 0.0
        self.ln_pair, self.ln_out = _LN(d), _LN(2 * d)
        for n in ("to_left", "to_left_gate", "to_right", "to_right_gate"):
            setattr(self, n, nn.Linear(d, 2 * d, bias=False))
        self.to_gate, self.to_out = nn.Linear(d, d, bias=False), nn.Linear(2 * d, d, bias=False)


def _same_parameters(a, b):
    sa, sb = a.state_dict(), b.state_dict()
    assert set(sa) == set(sb)
    for k in sa:
        assert torch.equal(sa[k].float(), sb[k].float()), k


def test_from_reference_keeps_parameters_direction_and_mode():
    ref = TriangleMultiplication(32, outgoing=False).eval()
    twin = from_reference(ref)
    assert isinstance(twin, TriangleMultiplicationB200) and twin.outgoing is False and not twin.training
    assert twin.p_drop == 0.25 and twin.ln_pair.eps == 1e-6 and twin.ln_out.eps == 1e-5
    _same_parameters(ref, twin)
    bi = from_reference(BidirectionalTriangleMultiplication(16))
    assert isinstance(bi, BidirectionalTriangleMultiplicationB200) and bi.d_hidden == 16 and bi.training
    assert bi.to_out.weight.shape == (16, 32)
    with pytest.raises(TypeError):
        from_reference(nn.Linear(4, 4))


def test_install_replaces_the_blocks_inside_a_model():
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.tri_out = TriangleMultiplication(16, True)
            self.tri_in = TriangleMultiplication(16, False)
            self.bidir = BidirectionalTriangleMultiplication(16)
            self.other = nn.Linear(16, 16)

    model = nn.Sequential(Block(), Block())
    before = [m for m in model.modules() if isinstance(m, (TriangleMultiplication, BidirectionalTriangleMultiplication))]
    assert install(model) == 6
    assert not any(isinstance(m, (TriangleMultiplication, BidirectionalTriangleMultiplication)) for m in model.modules())
    twins = [m for m in model.modules() if isinstance(m, (TriangleMultiplicationB200, BidirectionalTriangleMultiplicationB200))]
    assert len(twins) == 6
    for ref, twin in zip(before, twins):
        _same_parameters(ref, twin)
    assert isinstance(model[0].other, nn.Linear) and install(model) == 0


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="reference tree not present on this machine")
def test_from_reference_on_the_real_reference_modules():
    sys.path.insert(0, REFERENCE)
    try:
        from miniworld_engine.modules.triangle_multiplication.bidirectional import BidirectionalTriangleMultiplication as RefBi
        from miniworld_engine.modules.triangle_multiplication.reference import TriangleMultiplicationReference as RefUni
    finally:
        sys.path.remove(REFERENCE)
    uni = RefUni(32, outgoing=True)
    twin = from_reference(uni)
    assert isinstance(twin, TriangleMultiplicationB200) and twin.outgoing
    _same_parameters(uni, twin)
    bi = RefBi(32).to(torch.bfloat16)
    tb = from_reference(bi)
    assert isinstance(tb, BidirectionalTriangleMultiplicationB200)
    assert tb.to_left.weight.dtype == torch.bfloat16 and tb.ln_out.weight.dtype == torch.float32
    _same_parameters(bi, tb)
