"""Functional entry points of the B200 TriangleMultiplication block.

``triangle_multiplicative_update_b200`` has the signature of the reference's
functional interface (``src/miniworld_engine/modules/triangle_multiplication/interface.py:8-22``,
ground truth ``reference.py:86-122``, shipped op ``kernels/trimul_inproj/whole_op.py:170-184``)
and runs the three CUDA stages through the C-ABI library.  PyTorch is used for device
memory, streams and nothing else.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib

__all__ = [
    "triangle_multiplicative_update_b200",
    "trimul_forward",
    "read_status",
    "workspace_bytes",
]

_TORCH_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_FP32}

_workspaces: dict = {}
_status: dict = {}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _TORCH_DTYPES[t.dtype]
    except KeyError:
        raise NotImplementedError(
            f"trimul_b200 supports torch.bfloat16 and torch.float32 activations, got {t.dtype}") from None


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} must live on a CUDA device: trimul_b200 has no CPU path (got device {t.device})")


def _require_no_grad(what: str, *tensors) -> None:
    """The kernels have no backward.  The reference's functional op is autograd-transparent
    (``kernels/trimul_inproj/whole_op.py:170-190``) and its module routes grad-enabled calls to an
    autograd-capable path (``module.py:229-233``), so a caller that expects gradients must not be
    handed a silently detached result: raise instead."""
    if torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in tensors):
        raise NotImplementedError(
            f"{what} is forward-only (no backward kernels): call it under torch.no_grad(), or with "
            "inputs and parameters that do not require grad")


def _mask_bytes(mask: torch.Tensor) -> torch.Tensor:
    """Mask as one byte per element, without a kernel launch when it already is bool/uint8."""
    if mask.dtype == torch.bool:
        return mask.contiguous().view(torch.uint8)
    if mask.dtype == torch.uint8:
        return mask.contiguous()
    return (mask != 0).contiguous().view(torch.uint8)


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Grow-only per-(device, stream) scratch buffer for the a/b/tri planes."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _status_words(device: torch.device) -> torch.Tensor:
    st = _status.get(device.index)
    if st is None:
        st = torch.zeros(4, dtype=torch.int32, device=device)
        _status[device.index] = st
    return st


def read_status(device=None) -> tuple:
    """Synchronise and return the 4 device status words ``(code, stage, block, detail)``.
    ``code == 0`` means no bounded wait has expired since the words were created."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _status_words(device)
    torch.cuda.synchronize(device)
    return tuple(int(v) for v in st.cpu())


def workspace_bytes(B: int, N: int, c: int, dtype: torch.dtype, outgoing: bool = True) -> int:
    d = _lib.make_desc(B, N, c, dtype=_TORCH_DTYPES[dtype],
                       direction=_lib.OUTGOING if outgoing else _lib.INCOMING)
    n = C.c_size_t()
    _lib.check(_lib.load().trimul_b200_workspace_bytes(C.byref(d), C.byref(n), None, None, None),
               "trimul_b200_workspace_bytes")
    return n.value


_struct_cache: dict = {}
_STRUCT_CACHE_MAX = 256


def _pinned_weights(dtype, dims, specs):
    """``specs``: ten ``(tensor, name, expected shape)`` in the field order of ``trimul_weights``;
    1-D entries are the LayerNorm vectors (always fp32), 2-D ones Linear weights of ``dtype``.
    Validates, converts where dtype or layout differ, and returns ``(struct, copies)``: ``copies``
    are the conversions made here, which must outlive the enqueued kernels.

    A parameter set that needed no conversion is remembered under its addresses, dtypes, shapes and
    contiguity (all the struct depends on), so that the next call with the same parameters skips the
    validation: for the small problems a block call is otherwise bound by this host code."""
    key = [dtype, dims]
    for t, _, _ in specs:
        key += (t.data_ptr(), t.dtype, t.shape, t.is_contiguous())
    key = tuple(key)
    hit = _struct_cache.get(key)
    if hit is not None:
        return hit, []
    copies, ptrs = [], []
    for t, name, shape in specs:
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
        _require_cuda(t, name)
        want = torch.float32 if len(shape) == 1 else dtype
        if t.dtype != want or not t.is_contiguous():
            t = t.detach().to(want).contiguous()
            copies.append(t)
        ptrs.append(t.data_ptr())
    w = _lib.Weights(*ptrs)
    if not copies:
        if len(_struct_cache) >= _STRUCT_CACHE_MAX:
            _struct_cache.clear()
        _struct_cache[key] = w
    return w, copies


def _weights_struct(c, dtype, ln_in_w, ln_in_b, w_left, w_left_gate, w_right, w_right_gate,
                    ln_out_w, ln_out_b, w_gate, w_out, device, c_hidden=None, c_proj=None):
    """Validate and pin the parameter tensors; returns (struct, copies to keep alive).  ``c_hidden``
    (default ``c``) is the width of the output LayerNorm and the input width of ``to_out``;
    ``c_proj`` (default ``c``) the number of rows of the four input projections, i.e. the number
    of operand planes stage 1 produces per batch element."""
    h = c if c_hidden is None else c_hidden
    hp = c if c_proj is None else c_proj
    return _pinned_weights(dtype, (c, h, hp), (
        (ln_in_w, "norm_in_weight", (c,)), (ln_in_b, "norm_in_bias", (c,)),
        (w_left, "to_left.weight", (hp, c)), (w_left_gate, "to_left_gate.weight", (hp, c)),
        (w_right, "to_right.weight", (hp, c)), (w_right_gate, "to_right_gate.weight", (hp, c)),
        (ln_out_w, "norm_out_weight", (h,)), (ln_out_b, "norm_out_bias", (h,)),
        (w_gate, "to_gate.weight", (c, c)), (w_out, "to_out.weight", (c, h))))


def trimul_forward(
    x: torch.Tensor,
    mask: torch.Tensor | None,
    *,
    outgoing: bool,
    ln_in_weight, ln_in_bias, w_left, w_left_gate, w_right, w_right_gate,
    ln_out_weight, ln_out_bias, w_gate, w_out,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    residual: torch.Tensor | None = None,
    plain_kernels: bool = False,
    inplace_norm: bool = False,
    serial_launch: bool = False,
    drop_scale: torch.Tensor | None = None,
) -> torch.Tensor:
    """One block call on the current CUDA stream.  ``mask`` is a ``[B,N]`` token mask, a
    ``[B,N,N]`` pair mask or None; ``residual`` (same shape/dtype as ``x``) is added to the
    result when given.  Passing ``x`` itself as the residual (the block's ``pair + update`` form)
    costs nothing extra: the last stage adds the tile it already holds.  ``plain_kernels`` and
    ``inplace_norm`` select cross-checking variants of the kernels, ``serial_launch`` turns
    programmatic dependent launch of the stages off (see the flags in the C header).
    ``drop_scale`` is the reference module's row-broadcast dropout scale ``[B, 1, N, c]``
    (``module.py:332-337``): the block output is multiplied by it before the residual is added
    (``kernels/trimul_inproj/triton/gate_elem.py:41-78``).

    The hidden width ``h`` is read off the weights: the four input projections are ``[h, c]``,
    ``ln_out_*`` have ``h`` entries and ``w_out`` is ``[c, h]`` (``whole_op.py:203-209``).  bf16 with
    ``c = h = 128`` runs on the tensor-core kernels; any other multiple of 8 up to 256 runs stage 1
    (and, unless ``c = 128`` and ``h`` is 128 or 256, stage 3) on the warp-MMA kernels when both are
    multiples of 16 and the activations bf16, else on the CUDA-core kernels."""
    if x.dim() != 4 or x.shape[1] != x.shape[2]:
        raise ValueError(f"x must be [B, N, N, c], got {tuple(x.shape)}")
    _require_no_grad("trimul_forward", x, residual, ln_in_weight, ln_in_bias, w_left, w_left_gate, w_right,
                     w_right_gate, ln_out_weight, ln_out_bias, w_gate, w_out)
    _require_cuda(x, "x")
    B, N, _, c = x.shape
    code = _dtype_code(x)
    h = int(w_out.shape[-1])
    x = x.detach()
    if not x.is_contiguous():
        x = x.contiguous()
    mask_kind, mask_u8 = _lib.MASK_NONE, None
    if mask is not None:
        if tuple(mask.shape) == (B, N):
            mask_kind = _lib.MASK_TOKEN
        elif tuple(mask.shape) == (B, N, N):
            mask_kind = _lib.MASK_PAIR
        else:
            raise ValueError(f"mask must be [B,N] or [B,N,N], got {tuple(mask.shape)}")
        _require_cuda(mask, "mask")
        mask_u8 = _mask_bytes(mask)
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("residual must match x in shape and dtype")
        _require_cuda(residual, "residual")
        residual = residual.detach().contiguous()
    if drop_scale is not None:
        if tuple(drop_scale.shape) != (B, 1, N, c) or drop_scale.dtype != x.dtype:
            raise ValueError(f"drop_scale must be [B, 1, N, c] = {(B, 1, N, c)} of dtype {x.dtype}, got "
                             f"{tuple(drop_scale.shape)} {drop_scale.dtype}")
        _require_cuda(drop_scale, "drop_scale")
        drop_scale = drop_scale.detach().contiguous()

    lib = _lib.load()
    desc = _lib.make_desc(B, N, c, c_hidden=h, dtype=code, direction=_lib.OUTGOING if outgoing else _lib.INCOMING,
                          mask_kind=mask_kind, eps_in=eps_in, eps_out=eps_out,
                          flags=(_lib.FLAG_PLAIN_KERNELS if plain_kernels else 0) |
                          (_lib.FLAG_INPLACE_NORM_STAGE3 if inplace_norm else 0) |
                          (_lib.FLAG_SERIAL_LAUNCH if serial_launch else 0),
                          drop_scale=drop_scale.data_ptr() if drop_scale is not None else None)
    w, keep = _weights_struct(c, x.dtype, ln_in_weight, ln_in_bias, w_left, w_left_gate, w_right, w_right_gate,
                              ln_out_weight, ln_out_bias, w_gate, w_out, x.device, c_hidden=h, c_proj=h)
    nbytes = C.c_size_t()
    _lib.check(lib.trimul_b200_workspace_bytes(C.byref(desc), C.byref(nbytes), None, None, None),
               "trimul_b200_workspace_bytes")
    with torch.cuda.device(x.device):
        ws = _workspace(x.device, nbytes.value)
        out = torch.empty_like(x)
        st = _status_words(x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = lib.trimul_b200_forward(
            C.byref(desc), x.data_ptr(), mask_u8.data_ptr() if mask_u8 is not None else None, C.byref(w),
            out.data_ptr(), residual.data_ptr() if residual is not None else None,
            ws.data_ptr(), ws.numel(), stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_forward")
    # parameter copies made above must outlive the enqueued kernels
    for t in keep:
        t.record_stream(torch.cuda.current_stream(x.device))
    return out


def triangle_multiplicative_update_b200(
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
    """Drop-in for ``triangle_multiplicative_update_cute`` (``interface.py:8-22``).

    ``x (B,I,J,D)``; ``direction`` "outgoing" | "incoming" (anything else raises
    ``ValueError`` like ``reference.py:118-119``); ``mask`` a ``(B,I,J)`` pair mask, a
    ``(B,L)`` token mask (accepted by the shipped op, ``whole_op.py:56-58``) or None;
    ``p_in_weight (2H,D) = [to_left; to_right]``, ``g_in_weight (2H,D) = [to_left_gate;
    to_right_gate]``, ``norm_out_* (H,)``, ``p_out_weight (D,H) = to_out.weight``,
    ``g_out_weight (D,D) = to_gate.weight``; ``H = d_hidden`` is read off ``p_in_weight`` and an
    odd leading dimension raises ``ValueError`` (``whole_op.py:203-209``).  No residual is added.
    """
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be outgoing|incoming, got {direction!r}")
    two_h, d_in = int(p_in_weight.shape[0]), x.shape[-1]
    if two_h % 2 != 0:
        raise ValueError(f"p_in_weight leading dim must be 2*d_hidden (even), got {two_h}")
    D = two_h // 2
    if tuple(p_in_weight.shape) != (two_h, d_in) or tuple(g_in_weight.shape) != (two_h, d_in):
        raise ValueError(f"p_in_weight and g_in_weight must be ({two_h}, {d_in})")
    return trimul_forward(
        x, mask, outgoing=(direction == "outgoing"),
        ln_in_weight=norm_in_weight, ln_in_bias=norm_in_bias,
        w_left=p_in_weight[:D], w_left_gate=g_in_weight[:D],
        w_right=p_in_weight[D:], w_right_gate=g_in_weight[D:],
        ln_out_weight=norm_out_weight, ln_out_bias=norm_out_bias,
        w_gate=g_out_weight, w_out=p_out_weight, eps_in=eps, eps_out=eps)
