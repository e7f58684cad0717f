"""Stage-level entry points (LayerNorm+projections, contraction, output stage) on torch
tensors.  They expose the three C-ABI stage calls so that each kernel can be checked on
its own and so that the row-sharded multi-GPU driver can put collectives between them.

Operand planes are plain torch tensors plus a ``PlaneSpec`` that says how the logical
``[planes][rows][cols]`` array is laid out in them (see ``trimul_planes`` in
``include/trimul_b200.h``).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from .functional import _dtype_code, _mask_bytes, _require_cuda, _status_words, _weights_struct

__all__ = ["PlaneSpec", "alloc_planes", "planes_to_dense", "dense_to_planes", "tm1", "contract", "tm2", "round_up"]


def round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


@dataclass
class PlaneSpec:
    """Layout of channel-major planes inside ``buf`` (a flat or shaped tensor of the plane dtype)."""

    buf: torch.Tensor
    planes: int
    rows: int
    cols: int
    pitch: int
    plane_stride: int
    chunk_stride: int = 0
    row_chunk: int | None = None
    col_chunk: int | None = None

    def struct(self) -> _lib.Planes:
        return _lib.Planes(self.buf.data_ptr(), self.rows, self.cols, self.pitch, self.plane_stride,
                           self.chunk_stride,
                           self.rows if self.row_chunk is None else self.row_chunk,
                           self.cols if self.col_chunk is None else self.col_chunk)


def alloc_planes(planes: int, rows: int, cols: int, dtype: torch.dtype, device, *, fill=None,
                 row_chunk: int | None = None, col_chunk: int | None = None) -> PlaneSpec:
    """Allocate planes in the plain layout, or in the chunk-major layout an all-gather of
    per-rank slabs produces: ``[chunk][plane][rows_in_chunk][pitch]`` (row chunks) or
    ``[chunk][plane][rows][pitch_of_chunk]`` (column chunks)."""
    if row_chunk is not None and col_chunk is not None:
        raise ValueError("at most one of row_chunk / col_chunk")
    if row_chunk is not None:
        nchunk, r, cdim = -(-rows // row_chunk), row_chunk, cols
    elif col_chunk is not None:
        nchunk, r, cdim = -(-cols // col_chunk), rows, col_chunk
    else:
        nchunk, r, cdim = 1, rows, cols
    pitch = round_up(cdim, 8)
    plane_stride = r * pitch
    chunk_stride = planes * plane_stride
    buf = torch.empty(nchunk * chunk_stride, dtype=dtype, device=device)
    if fill is not None:
        buf.fill_(fill)
    return PlaneSpec(buf, planes, rows, cols, pitch, plane_stride, chunk_stride if nchunk > 1 else 0,
                     row_chunk, col_chunk)


def planes_to_dense(spec: PlaneSpec) -> torch.Tensor:
    """Gather the logical ``[planes, rows, cols]`` array out of a PlaneSpec (test helper)."""
    if spec.row_chunk is not None and spec.row_chunk < spec.rows:
        n = -(-spec.rows // spec.row_chunk)
        v = spec.buf[: n * spec.chunk_stride].view(n, spec.planes, spec.row_chunk, spec.pitch)[..., :spec.cols]
        return v.permute(1, 0, 2, 3).reshape(spec.planes, n * spec.row_chunk, spec.cols)[:, :spec.rows]
    if spec.col_chunk is not None and spec.col_chunk < spec.cols:
        n = -(-spec.cols // spec.col_chunk)
        v = spec.buf[: n * spec.chunk_stride].view(n, spec.planes, spec.rows, spec.pitch)[..., :spec.col_chunk]
        return v.permute(1, 2, 0, 3).reshape(spec.planes, spec.rows, n * spec.col_chunk)[..., :spec.cols]
    return spec.buf[: spec.planes * spec.plane_stride].view(spec.planes, spec.rows, spec.pitch)[..., :spec.cols]


def dense_to_planes(spec: PlaneSpec, dense: torch.Tensor) -> None:
    """Scatter a logical ``[planes, rows, cols]`` array into a PlaneSpec (test helper; chunked
    layouts need rows / cols to be whole multiples of the chunk size)."""
    P = spec.planes
    if spec.row_chunk is not None and spec.row_chunk < spec.rows:
        n = spec.rows // spec.row_chunk
        v = spec.buf[: n * spec.chunk_stride].view(n, P, spec.row_chunk, spec.pitch)[..., :spec.cols]
        v.permute(1, 0, 2, 3).copy_(dense.reshape(P, n, spec.row_chunk, spec.cols))
    elif spec.col_chunk is not None and spec.col_chunk < spec.cols:
        n = spec.cols // spec.col_chunk
        v = spec.buf[: n * spec.chunk_stride].view(n, P, spec.rows, spec.pitch)[..., :spec.col_chunk]
        v.permute(1, 2, 0, 3).copy_(dense.reshape(P, spec.rows, n, spec.col_chunk))
    else:
        spec.buf[: P * spec.plane_stride].view(P, spec.rows, spec.pitch)[..., :spec.cols].copy_(dense)


def _desc(x, N, outgoing, mask_kind, eps_in, eps_out, plain, row0, single_cta=False, inplace_norm=False,
          c_hidden=None, serial_launch=False):
    B, rows, _, c = x.shape
    return _lib.make_desc(B, N, c, c_hidden=c_hidden, dtype=_dtype_code(x),
                          direction=_lib.OUTGOING if outgoing else _lib.INCOMING, mask_kind=mask_kind,
                          eps_in=eps_in, eps_out=eps_out,
                          flags=(_lib.FLAG_PLAIN_KERNELS if plain else 0) |
                          (_lib.FLAG_SINGLE_CTA_STAGE1 if single_cta else 0) |
                          (_lib.FLAG_INPLACE_NORM_STAGE3 if inplace_norm else 0) |
                          (_lib.FLAG_SERIAL_LAUNCH if serial_launch else 0),
                          rows=rows, row0=row0)


def _mask_arg(mask, B, N):
    if mask is None:
        return _lib.MASK_NONE, None
    if tuple(mask.shape) == (B, N):
        kind = _lib.MASK_TOKEN
    elif tuple(mask.shape) == (B, N, N):
        kind = _lib.MASK_PAIR
    else:
        raise ValueError(f"mask must be [B,N] or [B,N,N] over the FULL token range, got {tuple(mask.shape)}")
    return kind, _mask_bytes(mask)


def tm1(z_slab: torch.Tensor, mask, weights: dict, a: PlaneSpec, b: PlaneSpec, *, outgoing: bool,
        row0: int = 0, eps: float = 1e-5, plain_kernels: bool = False, single_cta: bool = False,
        serial_launch: bool = False) -> None:
    """Stage 1 on a ``[B, rows, N, c]`` slab of z (rows ``row0 .. row0+rows`` of the grid).
    ``single_cta`` selects the lone-CTA form of the tensor-core kernel instead of the CTA-pair one;
    ``serial_launch`` (on every stage) turns programmatic dependent launch off."""
    _require_cuda(z_slab, "z")
    B, rows, N, c = z_slab.shape
    kind, mask_u8 = _mask_arg(mask, B, N)
    hp = int(weights["w_left"].shape[0])      # operand planes per batch element (d_hidden)
    d = _desc(z_slab, N, outgoing, kind, eps, eps, plain_kernels, row0, single_cta, c_hidden=hp,
              serial_launch=serial_launch)
    w, keep = _weights_struct(c, z_slab.dtype, device=z_slab.device, c_proj=hp,
                              c_hidden=int(weights["w_out"].shape[1]), **weights)
    st = _status_words(z_slab.device)
    with torch.cuda.device(z_slab.device):
        rc = _lib.load().trimul_b200_tm1(
            C.byref(d), z_slab.data_ptr(), mask_u8.data_ptr() if mask_u8 is not None else None, C.byref(w),
            C.byref(a.struct()), C.byref(b.struct()),
            torch.cuda.current_stream(z_slab.device).cuda_stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_tm1")
    for t in keep:
        t.record_stream(torch.cuda.current_stream(z_slab.device))


def contract(a: PlaneSpec, b: PlaneSpec, tri: PlaneSpec, *, plain_kernels: bool = False,
             single_cta: bool = False, serial_launch: bool = False) -> None:
    """Stage 2: ``tri[p] = a[p] @ b[p]^T`` for every plane."""
    dev = a.buf.device
    code = _lib.DTYPE_BF16 if a.buf.dtype == torch.bfloat16 else _lib.DTYPE_FP32
    st = _status_words(dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trimul_b200_contract(
            code, (_lib.FLAG_PLAIN_KERNELS if plain_kernels else 0) |
            (_lib.FLAG_SINGLE_CTA_CONTRACT if single_cta else 0) |
            (_lib.FLAG_SERIAL_LAUNCH if serial_launch else 0), a.planes,
            C.byref(a.struct()), C.byref(b.struct()), C.byref(tri.struct()),
            torch.cuda.current_stream(dev).cuda_stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_contract")


def _plane_array(specs):
    arr = (_lib.Planes * len(specs))()
    for k, sp in enumerate(specs):
        arr[k] = sp.struct()
    return arr


def tm1_scatter(z_slab: torch.Tensor, mask, weights: dict, a_dest, b_dest, *, outgoing: bool,
                row0: int = 0, eps: float = 1e-5) -> None:
    """Stage 1 whose output planes are split evenly over ``len(a_dest)`` destination buffers
    (``a_dest[k]`` / ``b_dest[k]`` receive planes ``[k*P, (k+1)*P)``); the buffers may be another
    GPU's memory mapped into this process.  Raises ``NotImplementedError`` where only the
    non-scattering stage exists (fp32, c != 128, odd plane counts)."""
    _require_cuda(z_slab, "z")
    B, rows, N, c = z_slab.shape
    kind, mask_u8 = _mask_arg(mask, B, N)
    d = _desc(z_slab, N, outgoing, kind, eps, eps, False, row0)
    w, keep = _weights_struct(c, z_slab.dtype, device=z_slab.device, **weights)
    st = _status_words(z_slab.device)
    if len(a_dest) != len(b_dest):
        raise ValueError("a_dest and b_dest must have the same length")
    aa, bb = _plane_array(a_dest), _plane_array(b_dest)
    with torch.cuda.device(z_slab.device):
        rc = _lib.load().trimul_b200_tm1_scatter(
            C.byref(d), z_slab.data_ptr(), mask_u8.data_ptr() if mask_u8 is not None else None, C.byref(w),
            len(a_dest), aa, bb, torch.cuda.current_stream(z_slab.device).cuda_stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_tm1_scatter")
    for t in keep:
        t.record_stream(torch.cuda.current_stream(z_slab.device))


def contract_scatter(a: PlaneSpec, b: PlaneSpec, tri_dest) -> None:
    """Stage 2 whose output rows are split evenly over ``len(tri_dest)`` destination buffers
    (``tri_dest[k]`` receives rows ``[k*R, (k+1)*R)``)."""
    dev = a.buf.device
    st = _status_words(dev)
    tt = _plane_array(tri_dest)
    with torch.cuda.device(dev):
        rc = _lib.load().trimul_b200_contract_scatter(
            _lib.DTYPE_BF16 if a.buf.dtype == torch.bfloat16 else _lib.DTYPE_FP32, 0, a.planes,
            C.byref(a.struct()), C.byref(b.struct()), len(tri_dest), tt,
            torch.cuda.current_stream(dev).cuda_stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_contract_scatter")


def tm2(z_slab: torch.Tensor, tri: PlaneSpec, weights: dict, *, residual=None, row0: int = 0,
        eps_in: float = 1e-5, eps_out: float = 1e-5, plain_kernels: bool = False,
        inplace_norm: bool = False, serial_launch: bool = False) -> torch.Tensor:
    """Stage 3 on a ``[B, rows, N, c]`` slab; returns the matching output slab.  The hidden width
    is read off ``weights["w_out"]`` (``[c, c_hidden]``): ``c``, or ``2c`` for the bidirectional
    block, whose ``tri`` holds ``B * 2c`` planes (per batch: outgoing planes, then incoming)."""
    _require_cuda(z_slab, "z")
    B, rows, N, c = z_slab.shape
    h = int(weights["w_out"].shape[1])
    d = _desc(z_slab, N, True, _lib.MASK_NONE, eps_in, eps_out, plain_kernels, row0, False, inplace_norm,
              c_hidden=h, serial_launch=serial_launch)
    w, keep = _weights_struct(c, z_slab.dtype, device=z_slab.device, c_hidden=h,
                              c_proj=int(weights["w_left"].shape[0]), **weights)
    out = torch.empty_like(z_slab)
    st = _status_words(z_slab.device)
    with torch.cuda.device(z_slab.device):
        rc = _lib.load().trimul_b200_tm2(
            C.byref(d), z_slab.data_ptr(), C.byref(tri.struct()), C.byref(w), out.data_ptr(),
            residual.data_ptr() if residual is not None else None,
            torch.cuda.current_stream(z_slab.device).cuda_stream, st.data_ptr())
    _lib.check(rc, "trimul_b200_tm2")
    for t in keep:
        t.record_stream(torch.cuda.current_stream(z_slab.device))
    return out
