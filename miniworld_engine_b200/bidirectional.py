"""Bidirectional TriangleMultiplication block on the B200 kernels.

Mirror of the reference's ``BidirectionalTriangleMultiplication``
(``src/miniworld_engine/modules/triangle_multiplication/bidirectional.py:34-156``): one input
LayerNorm, left/right gated projections of width ``2h`` (rows ``[:h]`` of each weight feed an
OUTGOING contraction, rows ``[h:]`` an INCOMING one), one LayerNorm over the ``2h`` concatenated
result channels, ``to_out: 2h -> d`` gated by ``to_gate(x_n)``, residual always added.

It is assembled from the stage entry points of the C-ABI library (``include/trimul_b200.h``):

* stage 1 runs twice per batch element, once per direction, each call with its half of the
  projection weights (a contiguous row block of the ``[2h, d]`` matrices) and writing its ``h``
  planes of the shared ``a`` / ``b`` plane sets — for the incoming half the kernel's strided TMA
  box stores the operands transposed, so
* stage 2 is ONE contraction over all ``B * 2h`` planes, and
* stage 3 is the wide form of the last stage (``c_hidden = 2c``): LayerNorm over ``2h`` channels
  folded into a ``[d, 2h]`` projection, the tri tile consumed as two 128-channel halves.

bf16 with ``d = h = 128`` takes the tensor-core kernels in every stage; other widths and fp32 take
the CUDA-core kernels (``2h <= 256``).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import stages as S
from .module import PinnedLayerNormParams

__all__ = ["bidir_trimul_forward", "BidirectionalTriangleMultiplicationB200"]


@torch.no_grad()
def bidir_trimul_forward(
    x: torch.Tensor,
    mask: torch.Tensor | None,
    *,
    ln_in_weight, ln_in_bias, w_left, w_left_gate, w_right, w_right_gate,
    ln_out_weight, ln_out_bias, w_gate, w_out,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    add_residual: bool = True,
    plain_kernels: bool = False,
) -> torch.Tensor:
    """``x + bidir_trimul(x)`` (or without the residual) on the current CUDA stream.

    ``x`` is ``[B, N, N, d]``; ``mask`` a ``[B, N]`` token mask or None; the four input
    projection weights are ``[2h, d]``, ``ln_out_*`` have ``2h`` entries, ``w_gate`` is ``[d, d]``
    and ``w_out`` ``[d, 2h]`` (``bidirectional.py:73-84``)."""
    if x.dim() != 4 or x.shape[1] != x.shape[2]:
        raise ValueError(f"x must be [B, N, N, d], got {tuple(x.shape)}")
    B, N, _, d = x.shape
    h2 = int(w_left.shape[0])
    if h2 % 2 or any(tuple(t.shape) != (h2, d) for t in (w_left, w_left_gate, w_right, w_right_gate)):
        raise ValueError("the four input projection weights must all be [2h, d]")
    h = h2 // 2
    if h != d:
        # the stage-1 kernels produce as many planes as z has channels
        raise NotImplementedError(f"d_hidden ({h}) != d_pair ({d}) is not supported")
    if tuple(w_out.shape) != (d, h2) or tuple(w_gate.shape) != (d, d):
        raise ValueError(f"w_out must be [{d}, {h2}] and w_gate [{d}, {d}]")
    if mask is not None and tuple(mask.shape) != (B, N):
        raise ValueError(f"mask must be [B, N], got {tuple(mask.shape)}")
    x = x.detach().contiguous()
    dev, dt = x.device, x.dtype
    cast = lambda t: t.detach().to(dt).contiguous()
    w_left, w_left_gate, w_right, w_right_gate = map(cast, (w_left, w_left_gate, w_right, w_right_gate))
    w_gate, w_out = cast(w_gate), cast(w_out)

    planes = B * h2
    a = S.alloc_planes(planes, N, N, dt, dev)
    b = S.alloc_planes(planes, N, N, dt, dev)
    tri = S.alloc_planes(planes, N, N, dt, dev)
    for bi in range(B):
        zb = x[bi:bi + 1]
        mb = None if mask is None else mask[bi:bi + 1]
        for direction in (0, 1):          # 0: outgoing half, 1: incoming half
            rows = slice(direction * h, (direction + 1) * h)
            first = (bi * h2 + direction * h) * a.plane_stride
            view = lambda spec: S.PlaneSpec(spec.buf[first:], h, N, N, spec.pitch, spec.plane_stride)
            # stage 1 reads only the input-side parameters; the output-side slots get placeholders
            wd = dict(ln_in_w=ln_in_weight, ln_in_b=ln_in_bias, w_left=w_left[rows], w_left_gate=w_left_gate[rows],
                      w_right=w_right[rows], w_right_gate=w_right_gate[rows], ln_out_w=ln_in_weight,
                      ln_out_b=ln_in_bias, w_gate=w_gate, w_out=w_gate)
            S.tm1(zb, mb, wd, view(a), view(b), outgoing=(direction == 0), eps=eps_in, plain_kernels=plain_kernels)
    S.contract(a, b, tri, plain_kernels=plain_kernels)
    wd3 = dict(ln_in_w=ln_in_weight, ln_in_b=ln_in_bias, w_left=w_gate, w_left_gate=w_gate, w_right=w_gate,
               w_right_gate=w_gate, ln_out_w=ln_out_weight, ln_out_b=ln_out_bias, w_gate=w_gate, w_out=w_out)
    return S.tm2(x, tri, wd3, residual=x if add_residual else None, eps_in=eps_in, eps_out=eps_out,
                 plain_kernels=plain_kernels)


class BidirectionalTriangleMultiplicationB200(nn.Module):
    """Drop-in for the reference's ``BidirectionalTriangleMultiplication`` (same constructor
    arguments that matter here, parameter names and ``state_dict`` keys,
    ``bidirectional.py:45-84``).  Forward-only."""

    def __init__(self, d_pair: int = 128, d_hidden: int | None = None, *, p_drop: float = 0.0):
        super().__init__()
        self.d_pair = d_pair
        self.d_hidden = d_pair if d_hidden is None else d_hidden
        self.p_drop = p_drop
        d2 = 2 * self.d_hidden
        self.ln_pair = PinnedLayerNormParams(d_pair)
        self.to_left = nn.Linear(d_pair, d2, bias=False)
        self.to_left_gate = nn.Linear(d_pair, d2, bias=False)
        self.to_right = nn.Linear(d_pair, d2, bias=False)
        self.to_right_gate = nn.Linear(d_pair, d2, bias=False)
        self.ln_out = PinnedLayerNormParams(d2)
        self.to_gate = nn.Linear(d_pair, d_pair, bias=False)
        self.to_out = nn.Linear(d2, d_pair, bias=False)
        with torch.no_grad():      # the reference zero-initialises the gates and to_out (bidirectional.py:78-84)
            for lin in (self.to_left_gate, self.to_right_gate, self.to_gate, self.to_out):
                lin.weight.zero_()

    @torch.no_grad()
    def block(self, pair: torch.Tensor, mask: torch.Tensor | None = None, *, add_residual: bool = True,
              plain_kernels: bool = False) -> torch.Tensor:
        return bidir_trimul_forward(
            pair, mask,
            ln_in_weight=self.ln_pair.weight, ln_in_bias=self.ln_pair.bias,
            w_left=self.to_left.weight, w_left_gate=self.to_left_gate.weight,
            w_right=self.to_right.weight, w_right_gate=self.to_right_gate.weight,
            ln_out_weight=self.ln_out.weight, ln_out_bias=self.ln_out.bias,
            w_gate=self.to_gate.weight, w_out=self.to_out.weight,
            eps_in=self.ln_pair.eps, eps_out=self.ln_out.eps,
            add_residual=add_residual, plain_kernels=plain_kernels)

    def forward(self, pair: torch.Tensor, mask: torch.Tensor | None = None,
                dropout_p: float | None = None) -> torch.Tensor:
        """``pair + drop_row(bidir_trimul(pair))`` (``bidirectional.py:93-156``)."""
        if torch.is_grad_enabled() and (pair.requires_grad or any(p.requires_grad for p in self.parameters())):
            raise NotImplementedError(
                "BidirectionalTriangleMultiplicationB200 is forward-only; wrap the call in torch.no_grad()")
        dropout_p = self.p_drop if dropout_p is None else dropout_p
        if dropout_p and dropout_p > 0.0 and self.training:
            b, _, l2, d = pair.shape      # row-broadcast dropout scale [B,1,L,D], bidirectional.py:86-91
            keep = torch.rand(b, 1, l2, d, device=pair.device, dtype=pair.dtype) > dropout_p
            return self.block(pair, mask, add_residual=False) * (keep.to(pair.dtype) / (1.0 - dropout_p)) + pair
        return self.block(pair, mask)
