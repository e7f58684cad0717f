"""Bidirectional TriangleMultiplication block on the B200 kernels.

Mirror of the reference's ``BidirectionalTriangleMultiplication``
(``src/miniworld_engine/modules/triangle_multiplication/bidirectional.py:34-156``): one input
LayerNorm, left/right gated projections of width ``2h`` (rows ``[:h]`` of each weight feed an
OUTGOING contraction, rows ``[h:]`` an INCOMING one), one LayerNorm over the ``2h`` concatenated
result channels, ``to_out: 2h -> d`` gated by ``to_gate(x_n)``, residual always added.

``trimul_b200_forward_bidir`` of the C-ABI library (``include/trimul_b200.h``) assembles it from
the stage entry points:

* stage 1 runs twice per batch element, once per direction, each call with its half of the
  projection weights (a contiguous row block of the ``[2h, d]`` matrices) and writing its ``h``
  planes of the shared ``a`` / ``b`` plane sets — for the incoming half the kernel's strided TMA
  box stores the operands transposed, so
* stage 2 is ONE contraction over all ``B * 2h`` planes, and
* stage 3 is the last stage with ``c_hidden = 2h``: LayerNorm over ``2h`` channels folded into a
  ``[d, 2h]`` projection (for ``h = 128`` the tri tile is consumed as two 128-channel halves).

bf16 with ``d = h = 128`` takes the tensor-core kernels in every stage.  ``d_hidden != d_pair``
(``h`` a multiple of 8, ``2h <= 256``) is served too: stage 1 then runs on the warp-MMA kernel
(widths that are multiples of 16; otherwise the CUDA-core kernel),
the contraction stays on the tensor cores for bf16, and stage 3 does when ``d = 128`` and
``2h`` is 128 or 256.  fp32 takes the CUDA-core kernels throughout.

``bidirectional_triangle_multiplicative_update_b200`` is the same call under the argument names of
the reference's functional op (``kernels/trimul_inproj/whole_op.py:243-262``).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn

from . import _lib
from .functional import (_dtype_code, _mask_bytes, _pinned_weights, _require_cuda, _require_no_grad,
                         _status_words, _workspace)
from .module import PinnedLayerNormParams, _lecun_trunc_normal_

__all__ = ["bidir_trimul_forward", "bidirectional_triangle_multiplicative_update_b200",
           "BidirectionalTriangleMultiplicationB200"]


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
    if h2 % 16 or d % 8 or h2 > 256 or d > 256:
        raise NotImplementedError(
            f"d_pair ({d}) and d_hidden ({h2 // 2}) must be multiples of 8 with d_pair, 2*d_hidden <= 256")
    if tuple(w_out.shape) != (d, h2) or tuple(w_gate.shape) != (d, d):
        raise ValueError(f"w_out must be [{d}, {h2}] and w_gate [{d}, {d}]")
    if mask is not None and tuple(mask.shape) != (B, N):
        raise ValueError(f"mask must be [B, N], got {tuple(mask.shape)}")
    _require_no_grad("bidir_trimul_forward", x, ln_in_weight, ln_in_bias, w_left, w_left_gate, w_right, w_right_gate,
                     ln_out_weight, ln_out_bias, w_gate, w_out)
    _require_cuda(x, "x")
    x = x.detach().contiguous()
    mask_kind, mask_u8 = _lib.MASK_NONE, None
    if mask is not None:
        _require_cuda(mask, "mask")
        mask_kind, mask_u8 = _lib.MASK_TOKEN, _mask_bytes(mask)
    desc = _lib.make_desc(B, N, d, c_hidden=h2, dtype=_dtype_code(x), direction=_lib.OUTGOING, mask_kind=mask_kind,
                          eps_in=eps_in, eps_out=eps_out, flags=_lib.FLAG_PLAIN_KERNELS if plain_kernels else 0)
    w, keep = _bidir_weights_struct(d, h2, x.dtype, ln_in_weight, ln_in_bias, w_left, w_left_gate, w_right,
                                    w_right_gate, ln_out_weight, ln_out_bias, w_gate, w_out)
    lib = _lib.load()
    nbytes = C.c_size_t()
    _lib.check(lib.trimul_b200_bidir_workspace_bytes(C.byref(desc), C.byref(nbytes)),
               "trimul_b200_bidir_workspace_bytes")
    with torch.cuda.device(x.device):
        ws = _workspace(x.device, nbytes.value)
        out = torch.empty_like(x)
        st = _status_words(x.device)
        rc = lib.trimul_b200_forward_bidir(
            C.byref(desc), x.data_ptr(), mask_u8.data_ptr() if mask_u8 is not None else None, C.byref(w),
            out.data_ptr(), 1 if add_residual else 0, ws.data_ptr(), ws.numel(),
            torch.cuda.current_stream(x.device).cuda_stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_forward_bidir")
    for t in keep:      # parameter copies made above must outlive the enqueued kernels
        t.record_stream(torch.cuda.current_stream(x.device))
    return out


def bidirectional_triangle_multiplicative_update_b200(
    x: torch.Tensor,
    mask: torch.Tensor | None = None,
    *,
    norm_in_weight, norm_in_bias, to_left_weight, to_left_gate_weight, to_right_weight, to_right_gate_weight,
    norm_out_weight, norm_out_bias, to_out_weight, to_gate_weight,
    eps: float = 1e-5,
) -> torch.Tensor:
    """Drop-in for ``ops.bidirectional_triangle_multiplicative_update``
    (``kernels/trimul_inproj/whole_op.py:243-262``): ``x (B,L,L,d_pair)``, ``mask (B,L)`` or None, the
    four input projections ``(2*d_hidden, d_pair)``, ``norm_out_* (2*d_hidden,)``, ``to_out_weight
    (d_pair, 2*d_hidden)``, ``to_gate_weight (d_pair, d_pair)``.  Returns the update WITHOUT the
    residual, like the op it replaces (the module adds it)."""
    return bidir_trimul_forward(
        x, mask, ln_in_weight=norm_in_weight, ln_in_bias=norm_in_bias, w_left=to_left_weight,
        w_left_gate=to_left_gate_weight, w_right=to_right_weight, w_right_gate=to_right_gate_weight,
        ln_out_weight=norm_out_weight, ln_out_bias=norm_out_bias, w_gate=to_gate_weight, w_out=to_out_weight,
        eps_in=eps, eps_out=eps, add_residual=False)


def _bidir_weights_struct(d, h2, dtype, ln_in_w, ln_in_b, w_left, w_left_gate, w_right, w_right_gate,
                          ln_out_w, ln_out_b, w_gate, w_out):
    """Validate and pin the bidirectional block's parameters; returns (struct, copies to keep alive)."""
    return _pinned_weights(dtype, (d, h2, h2), (
        (ln_in_w, "ln_pair.weight", (d,)), (ln_in_b, "ln_pair.bias", (d,)),
        (w_left, "to_left.weight", (h2, d)), (w_left_gate, "to_left_gate.weight", (h2, d)),
        (w_right, "to_right.weight", (h2, d)), (w_right_gate, "to_right_gate.weight", (h2, d)),
        (ln_out_w, "ln_out.weight", (h2,)), (ln_out_b, "ln_out.bias", (h2,)),
        (w_gate, "to_gate.weight", (d, d)), (w_out, "to_out.weight", (d, h2))))


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
        with torch.no_grad():
            # the reference's "default" (LeCun truncated normal) init for the two projections and zeros
            # for the gates and to_out (bidirectional.py:77-84)
            _lecun_trunc_normal_(self.to_left.weight)
            _lecun_trunc_normal_(self.to_right.weight)
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
