"""CPU oracle for the TriangleMultiplication block.  TEST INFRASTRUCTURE ONLY.

This file is a from-scratch CPU restatement of the reference's ground-truth
algorithm.  It exists to check the CUDA path; it is never the thing shipped or
measured as the product.  Only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.
The product path (the package's C-ABI library) never routes through here.

Parity status: PINNED.  The restatement is compared against outputs of the
reference's own ``TriangleMultiplicationReference`` / functional twin on seeded
inputs; those outputs are committed as fixtures under ``tests/golden/`` together
with the script that generated them.

What is restated (paths are relative to the reference project root):

* whole block, module form
  ``src/miniworld_engine/modules/triangle_multiplication/reference.py:62-83``
* whole block, functional form with concatenated in-projection weights and a
  pair mask ``reference.py:86-122``
* LayerNorm: biased variance, computed in fp32 and cast back to the activation
  dtype, affine parameters kept in fp32 under any module cast
  ``src/miniworld_engine/modules/primitives.py:70-88,146-153``
* sigmoid gate ``src/miniworld_engine/modules/ops.py:11-16``
* bidirectional block, eager branch: doubled-width input projections, outgoing contraction on
  the first half of the hidden channels and incoming on the second, one LayerNorm over both,
  residual always added
  ``src/miniworld_engine/modules/triangle_multiplication/bidirectional.py:134-156``

Arithmetic notes that matter for parity:

* In bf16 mode every op boundary rounds to bf16 exactly as eager PyTorch does
  for a module cast with ``.to(torch.bfloat16)``: the LayerNorm output, each
  Linear output, the sigmoid, each product, the masked operands, the
  contraction output, the second LayerNorm output and the final product.
* The token mask becomes a pair mask ``m[i] & m[k]`` that multiplies the gated
  left/right operands only.  The output gate sees the *unmasked* normalised
  input (``reference.py:72-75,83``).
* No residual is added by the block itself (``reference.py:83``); the reference's
  kernel-backed module adds ``pair`` afterwards, after the optional row-broadcast
  dropout scale (``module.py:208-222``): ``trimul_module_forward`` restates that.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

__all__ = [
    "TrimulWeights",
    "make_weights",
    "make_input",
    "make_token_mask",
    "trimul_forward",
    "trimul_forward_functional",
    "trimul_stages",
    "make_bidir_weights",
    "bidir_forward",
    "rel_rms",
    "block_flops",
]


# --------------------------------------------------------------------------- #
# parameters
# --------------------------------------------------------------------------- #
@dataclass
class TrimulWeights:
    """Parameter set with the reference module's names (``reference.py:51-59``).

    Linear weights are ``[out_features, in_features]`` (``nn.Linear``), no bias.
    ``ln_*`` parameters are always fp32 (``primitives.py:70-88``).
    """

    ln_pair_weight: torch.Tensor
    ln_pair_bias: torch.Tensor
    to_left: torch.Tensor
    to_left_gate: torch.Tensor
    to_right: torch.Tensor
    to_right_gate: torch.Tensor
    ln_out_weight: torch.Tensor
    ln_out_bias: torch.Tensor
    to_gate: torch.Tensor
    to_out: torch.Tensor
    eps_in: float = 1e-5
    eps_out: float = 1e-5
    _linear_names: tuple = field(
        default=("to_left", "to_left_gate", "to_right", "to_right_gate", "to_gate", "to_out"),
        repr=False,
    )

    def to(self, dtype: torch.dtype) -> "TrimulWeights":
        """What ``module.to(dtype)`` does to the reference module's parameters.

        Linear weights are cast.  LayerNorm parameters remain fp32 *tensors*, but
        their values pass through ``dtype`` on the way: the reference's pinning
        hook applies the cast first and then widens the result back to fp32
        (``primitives.py:80-86``), so after ``.to(torch.bfloat16)`` gamma/beta hold
        bf16-representable values.
        """
        kw = {k: getattr(self, k).to(dtype).float() for k in (
            "ln_pair_weight", "ln_pair_bias", "ln_out_weight", "ln_out_bias")}
        for k in self._linear_names:
            kw[k] = getattr(self, k).to(dtype)
        return TrimulWeights(eps_in=self.eps_in, eps_out=self.eps_out, **kw)

    def state_dict(self) -> dict:
        """Keys of ``TriangleMultiplicationReference.state_dict()``."""
        return {
            "ln_pair.weight": self.ln_pair_weight,
            "ln_pair.bias": self.ln_pair_bias,
            "to_left.weight": self.to_left,
            "to_left_gate.weight": self.to_left_gate,
            "to_right.weight": self.to_right,
            "to_right_gate.weight": self.to_right_gate,
            "ln_out.weight": self.ln_out_weight,
            "ln_out.bias": self.ln_out_bias,
            "to_gate.weight": self.to_gate,
            "to_out.weight": self.to_out,
        }


def make_weights(c: int, seed: int = 0, *, affine: str = "unit", h: int | None = None) -> TrimulWeights:
    """Seeded synthetic weights.

    The six Linear weights are drawn in the fixed order ``to_left, to_left_gate,
    to_right, to_right_gate, to_gate, to_out`` as ``randn(c, c) * c**-0.5`` from a
    CPU generator (the benchmark harness of the reference overrides the library's
    zero-initialised gates the same way, ``benchmarks/runners/bench.py:550-563``).

    ``affine="unit"`` gives gamma=1, beta=0; ``affine="random"`` draws non-trivial
    LayerNorm parameters (after the Linear weights, so the Linear draws do not
    depend on this switch) to expose mask/gate ordering mistakes.

    ``h`` (default ``c``) is the hidden width of the functional op
    (``kernels/trimul_inproj/whole_op.py:203-209``): the four input projections become
    ``[h, c]``, ``ln_out`` gets ``h`` channels and ``to_out`` is ``[c, h]``; with ``h == c`` the
    draws are exactly those of the module form.
    """
    h = c if h is None else h
    g = torch.Generator().manual_seed(seed)
    lin = [torch.randn(h, c, generator=g) * c ** -0.5 for _ in range(4)]
    lin.append(torch.randn(c, c, generator=g) * c ** -0.5)
    lin.append(torch.randn(c, h, generator=g) * h ** -0.5)
    if affine == "unit":
        gi, bi, go, bo = torch.ones(c), torch.zeros(c), torch.ones(h), torch.zeros(h)
    elif affine == "random":
        gi = 1.0 + 0.3 * torch.randn(c, generator=g)
        bi = 0.2 * torch.randn(c, generator=g)
        go = 1.0 + 0.3 * torch.randn(h, generator=g)
        bo = 0.2 * torch.randn(h, generator=g)
    else:
        raise ValueError(f"affine must be unit|random, got {affine!r}")
    return TrimulWeights(gi, bi, lin[0], lin[1], lin[2], lin[3], go, bo, lin[4], lin[5])


def make_input(B: int, N: int, c: int, seed: int = 1) -> torch.Tensor:
    """``z ~ N(0,1)`` of shape ``[B, N, N, c]`` fp32 from a CPU generator."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, N, N, c, generator=g)


def make_token_mask(B: int, N: int, kind: str = "ones", seed: int = 2) -> torch.Tensor:
    """Token masks of the benchmark configurations.

    ``ones``; ``tail77`` (last 77 tokens padded); ``rand5`` (each token padded
    with probability 0.05, fixed by ``seed``); ``tail<k>`` for a general tail.
    """
    m = torch.ones(B, N, dtype=torch.bool)
    if kind == "ones":
        return m
    if kind.startswith("tail"):
        k = int(kind[4:])
        if k > 0:
            m[:, N - k:] = False
        return m
    if kind == "rand5":
        g = torch.Generator().manual_seed(seed)
        return torch.rand(B, N, generator=g) > 0.05
    raise ValueError(f"unknown mask kind {kind!r}")


# --------------------------------------------------------------------------- #
# the algorithm
# --------------------------------------------------------------------------- #
def _layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    # primitives.py:146-153: fp32 compute, cast back to the activation dtype.
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


def _gate(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    # ops.py:11-16
    return torch.sigmoid(g) * x


def trimul_stages(
    z: torch.Tensor,
    token_mask: torch.Tensor | None,
    w: TrimulWeights,
    outgoing: bool = True,
    pair_mask: torch.Tensor | None = None,
) -> dict:
    """All intermediates of the block, in the reference's row-major layout.

    Returns ``x_n, left, right`` (masked), ``tri`` (contraction), ``tri_n``
    (after the output LayerNorm) and ``out``; follows ``reference.py:66-83``.
    ``pair_mask`` ([B,N,N] bool) overrides the token mask (functional form,
    ``reference.py:108-111``).
    """
    x_n = _layer_norm(z, w.ln_pair_weight, w.ln_pair_bias, w.eps_in)
    left = _gate(F.linear(x_n, w.to_left_gate), F.linear(x_n, w.to_left))
    right = _gate(F.linear(x_n, w.to_right_gate), F.linear(x_n, w.to_right))
    if pair_mask is not None:
        m = pair_mask.to(left.dtype).unsqueeze(-1)
        left, right = left * m, right * m
    elif token_mask is not None:
        m2 = (token_mask.unsqueeze(-1) & token_mask.unsqueeze(-2)).unsqueeze(-1)
        left, right = left * m2, right * m2
    if outgoing:
        tri = torch.einsum("bikd,bjkd->bijd", left, right)
    else:
        tri = torch.einsum("bkid,bkjd->bijd", left, right)
    tri_n = _layer_norm(tri, w.ln_out_weight, w.ln_out_bias, w.eps_out)
    out = _gate(F.linear(x_n, w.to_gate), F.linear(tri_n, w.to_out))
    return {"x_n": x_n, "left": left, "right": right, "tri": tri, "tri_n": tri_n, "out": out}


@torch.no_grad()
def trimul_forward(
    z: torch.Tensor,
    token_mask: torch.Tensor | None,
    w: TrimulWeights,
    outgoing: bool = True,
) -> torch.Tensor:
    """Module-form block output (no residual), ``reference.py:62-83``."""
    return trimul_stages(z, token_mask, w, outgoing)["out"]


@torch.no_grad()
def trimul_module_forward(
    z: torch.Tensor,
    token_mask: torch.Tensor | None,
    w: TrimulWeights,
    outgoing: bool = True,
    drop_scale: torch.Tensor | None = None,
) -> torch.Tensor:
    """What the reference MODULE returns: ``pair + drop_row(trimul(pair))``
    (``src/miniworld_engine/modules/triangle_multiplication/module.py:208-222``): the block output,
    times the row-broadcast dropout scale ``[B, 1, N, c]`` when one is live (training,
    ``module.py:332-337``), plus the input.  Each step rounds to the activation dtype as eager
    PyTorch does."""
    out = trimul_stages(z, token_mask, w, outgoing)["out"]
    if drop_scale is not None:
        out = out * drop_scale
    return out + z


@torch.no_grad()
def trimul_forward_functional(
    x: torch.Tensor,
    direction: str,
    mask: torch.Tensor | None,
    norm_in_weight: torch.Tensor,
    norm_in_bias: torch.Tensor,
    p_in_weight: torch.Tensor,
    g_in_weight: torch.Tensor,
    norm_out_weight: torch.Tensor,
    norm_out_bias: torch.Tensor,
    p_out_weight: torch.Tensor,
    g_out_weight: torch.Tensor,
    eps: float = 1e-5,
) -> torch.Tensor:
    """Functional form with ``p_in = [to_left; to_right]``, ``g_in = [to_left_gate;
    to_right_gate]`` and a ``[B,I,J]`` pair mask, ``reference.py:86-122``.  The split point is
    the hidden width ``p_in_weight.shape[0] // 2`` as in the shipped op
    (``kernels/trimul_inproj/whole_op.py:203-209``); ``reference.py:99`` writes it as ``D`` and so
    only covers ``d_hidden == d_pair``."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be outgoing|incoming, got {direction!r}")
    D = p_in_weight.shape[0] // 2
    w = TrimulWeights(
        norm_in_weight, norm_in_bias,
        p_in_weight[:D], g_in_weight[:D], p_in_weight[D:], g_in_weight[D:],
        norm_out_weight, norm_out_bias, g_out_weight, p_out_weight,
        eps_in=eps, eps_out=eps,
    )
    return trimul_stages(x, None, w, direction == "outgoing", pair_mask=mask)["out"]


# --------------------------------------------------------------------------- #
# bidirectional block
# --------------------------------------------------------------------------- #
def make_bidir_weights(d: int, h: int | None = None, seed: int = 0, *, affine: str = "unit") -> TrimulWeights:
    """Seeded weights with the shapes of the reference's bidirectional module
    (``bidirectional.py:73-84``): ``to_left``, ``to_left_gate``, ``to_right``, ``to_right_gate``
    are ``[2h, d]`` (rows ``[:h]`` feed the outgoing contraction, ``[h:]`` the incoming one),
    ``ln_out`` has ``2h`` channels, ``to_gate`` is ``[d, d]`` and ``to_out`` ``[d, 2h]``.  Same
    field names as ``TrimulWeights``, so ``.to()`` and ``.state_dict()`` apply unchanged."""
    h = d if h is None else h
    g = torch.Generator().manual_seed(seed)
    lin = [torch.randn(2 * h, d, generator=g) * d ** -0.5 for _ in range(4)]
    to_gate = torch.randn(d, d, generator=g) * d ** -0.5
    to_out = torch.randn(d, 2 * h, generator=g) * (2 * h) ** -0.5
    if affine == "unit":
        gi, bi, go, bo = torch.ones(d), torch.zeros(d), torch.ones(2 * h), torch.zeros(2 * h)
    elif affine == "random":
        gi = 1.0 + 0.3 * torch.randn(d, generator=g)
        bi = 0.2 * torch.randn(d, generator=g)
        go = 1.0 + 0.3 * torch.randn(2 * h, generator=g)
        bo = 0.2 * torch.randn(2 * h, generator=g)
    else:
        raise ValueError(f"affine must be unit|random, got {affine!r}")
    return TrimulWeights(gi, bi, lin[0], lin[1], lin[2], lin[3], go, bo, to_gate, to_out)


@torch.no_grad()
def bidir_forward(z: torch.Tensor, token_mask: torch.Tensor | None, w: TrimulWeights,
                  add_residual: bool = True) -> torch.Tensor:
    """``pair + bidir_trimul(pair)`` as the eager branch of the reference computes it
    (``bidirectional.py:134-156``; the residual is unconditional there, ``:105-116``)."""
    h = w.to_left.shape[0] // 2
    x_n = _layer_norm(z, w.ln_pair_weight, w.ln_pair_bias, w.eps_in)
    left = _gate(F.linear(x_n, w.to_left_gate), F.linear(x_n, w.to_left))
    right = _gate(F.linear(x_n, w.to_right_gate), F.linear(x_n, w.to_right))
    if token_mask is not None:
        m2 = (token_mask.unsqueeze(-1) & token_mask.unsqueeze(-2)).unsqueeze(-1)
        left, right = left * m2, right * m2
    out_outgoing = torch.einsum("bikd,bjkd->bijd", left[..., :h], right[..., :h])
    out_incoming = torch.einsum("bkid,bkjd->bijd", left[..., h:], right[..., h:])
    tri = torch.cat([out_outgoing, out_incoming], dim=-1)
    tri_n = _layer_norm(tri, w.ln_out_weight, w.ln_out_bias, w.eps_out)
    out = _gate(F.linear(x_n, w.to_gate), F.linear(tri_n, w.to_out))
    return out + z if add_residual else out


# --------------------------------------------------------------------------- #
# metrics
# --------------------------------------------------------------------------- #
def rel_rms(y: torch.Tensor, ref: torch.Tensor) -> float:
    """``||y - ref||_2 / ||ref||_2`` in fp64 (the tolerance metric)."""
    y64, r64 = y.double(), ref.double()
    den = r64.norm().item()
    num = (y64 - r64).norm().item()
    return num / den if den > 0 else num


def block_flops(B: int, N: int, c: int) -> float:
    """Algorithmic FLOPs of one block call: contraction + six c x c projections
    (the reference's own accounting, ``docs/kernels/triangle-multiplication-module.md:42-49``)."""
    return float(B) * (2.0 * N ** 3 * c + 12.0 * N ** 2 * c ** 2)
