"""``nn.Module`` mirror of the reference's TriangleMultiplication for the B200 backend.

Same constructor, ``forward`` signature, parameter names/shapes and ``state_dict`` keys as
``src/miniworld_engine/modules/triangle_multiplication/module.py:94-103,192-197`` and
``reference.py:39-59``, so ``load_state_dict`` round-trips between the two.  ``forward``
returns ``pair + trimul(pair)`` like the reference module (``module.py:106-122,208``);
``TriangleMultiplicationB200.block`` returns the bare block output that ``reference.py``
defines (no residual).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import functional as F_b200

__all__ = ["TriangleMultiplicationB200", "PinnedLayerNormParams"]


class PinnedLayerNormParams(nn.Module):
    """LayerNorm affine parameters that stay fp32 tensors under any module cast.

    Mirrors the reference's pinning hook (``modules/primitives.py:70-88``): the cast is
    applied and the result widened back to fp32, so after ``.to(torch.bfloat16)`` the
    values are bf16-representable but the tensors remain fp32.
    """

    def __init__(self, dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.normalized_shape = (dim,)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.float32))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=torch.float32))

    def _apply(self, fn, *args, **kwargs):
        def fp32_fn(t):
            out = fn(t)
            if isinstance(out, torch.Tensor) and out.is_floating_point():
                out = out.to(torch.float32)
            return out

        return super()._apply(fp32_fn, *args, **kwargs)


def _lecun_trunc_normal_(w: torch.Tensor) -> None:
    """Fan-in truncated normal on [-2, 2] sigma with unit-variance correction — the
    reference's "default" Linear init (``modules/primitives.py:24-47``)."""
    fan_in = w.shape[1]
    # std of a standard normal truncated to [-2, 2]
    trunc_std = 0.8796256610342398
    std = math.sqrt(1.0 / max(1, fan_in)) / trunc_std
    nn.init.trunc_normal_(w, mean=0.0, std=std, a=-2.0 * std, b=2.0 * std)


class TriangleMultiplicationB200(nn.Module):
    """Triangular multiplicative update on the B200 kernels.

    Parameters follow the reference module: ``d_pair``; ``d_hidden`` (must equal ``d_pair``
    or be None — the reference's input projections are ``d_pair`` wide regardless,
    ``reference.py:51-59``); ``outgoing``; ``p_drop`` (row-broadcast dropout in training
    only, ``module.py:117-118``).  ``implementation`` / ``ln_implementation`` are accepted
    for signature compatibility and ignored: there is exactly one backend here.
    """

    def __init__(
        self,
        d_pair: int = 128,
        *,
        d_hidden: int | None = None,
        outgoing: bool = True,
        implementation=None,
        ln_implementation=None,
        p_drop: float = 0.0,
    ) -> None:
        super().__init__()
        if d_hidden is None:
            d_hidden = d_pair
        if d_hidden != d_pair:
            raise ValueError(
                f"d_hidden != d_pair ({d_hidden} != {d_pair}) is not supported by the B200 backend")
        self.outgoing = outgoing
        self.p_drop = p_drop
        self.implementation = "b200"
        self.ln_pair = PinnedLayerNormParams(d_pair)
        self.to_left = nn.Linear(d_pair, d_pair, bias=False)
        self.to_left_gate = nn.Linear(d_pair, d_pair, bias=False)
        self.to_right = nn.Linear(d_pair, d_pair, bias=False)
        self.to_right_gate = nn.Linear(d_pair, d_pair, bias=False)
        self.ln_out = PinnedLayerNormParams(d_pair)
        self.to_gate = nn.Linear(d_pair, d_pair, bias=False)
        self.to_out = nn.Linear(d_hidden, d_pair, bias=False)
        with torch.no_grad():
            _lecun_trunc_normal_(self.to_left.weight)
            _lecun_trunc_normal_(self.to_right.weight)
            for lin in (self.to_left_gate, self.to_right_gate, self.to_gate, self.to_out):
                lin.weight.zero_()

    @torch.no_grad()
    def block(self, pair: torch.Tensor, mask: torch.Tensor | None = None, *,
              residual: torch.Tensor | None = None, plain_kernels: bool = False,
              drop_scale: torch.Tensor | None = None) -> torch.Tensor:
        """The block output as ``reference.py:62-83`` defines it (no residual unless given;
        ``drop_scale`` ``[B, 1, L, D]`` multiplies it before the residual is added)."""
        return F_b200.trimul_forward(
            pair, mask, outgoing=self.outgoing,
            ln_in_weight=self.ln_pair.weight, ln_in_bias=self.ln_pair.bias,
            w_left=self.to_left.weight, w_left_gate=self.to_left_gate.weight,
            w_right=self.to_right.weight, w_right_gate=self.to_right_gate.weight,
            ln_out_weight=self.ln_out.weight, ln_out_bias=self.ln_out.bias,
            w_gate=self.to_gate.weight, w_out=self.to_out.weight,
            eps_in=self.ln_pair.eps, eps_out=self.ln_out.eps,
            residual=residual, plain_kernels=plain_kernels, drop_scale=drop_scale)

    def forward(self, pair: torch.Tensor, mask: torch.Tensor | None = None,
                dropout_p: float | None = None) -> torch.Tensor:
        """``pair + drop_row(trimul(pair))`` (``module.py:192-222``).  Forward-only: the
        kernels have no backward, so calling this under autograd with parameters that
        require grad raises instead of silently detaching."""
        if torch.is_grad_enabled() and (pair.requires_grad or any(p.requires_grad for p in self.parameters())):
            raise NotImplementedError(
                "TriangleMultiplicationB200 is forward-only; wrap the call in torch.no_grad()")
        dropout_p = self.p_drop if dropout_p is None else dropout_p
        if dropout_p and dropout_p > 0.0 and self.training:
            # row-broadcast dropout scale [B,1,L,D] = (rand > p) / (1 - p), module.py:332-337
            b, _, l2, d = pair.shape
            keep = torch.rand(b, 1, l2, d, device=pair.device, dtype=pair.dtype) > dropout_p
            # scale and residual are applied in the last stage's epilogue, like the reference's gate
            # kernel does (kernels/trimul_inproj/triton/gate_elem.py:41-78)
            return self.block(pair, mask, residual=pair, drop_scale=keep.to(pair.dtype) / (1.0 - dropout_p))
        return self.block(pair, mask, residual=pair)
