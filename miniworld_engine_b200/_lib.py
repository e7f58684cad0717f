"""ctypes binding of ``libtrimul_b200.so`` (the C ABI declared in ``include/trimul_b200.h``).

The library is the only compute path of this package.  If it is missing or cannot
be loaded, every entry point raises — there is no PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libtrimul_b200.so")

ABI_VERSION = 2

OK = 0
E_INVALID, E_UNSUPPORTED, E_WORKSPACE, E_CUDA, E_DEVICE_TIMEOUT = -1, -2, -3, -4, -5
E_STATIC_SCRATCH = -6
STATIC_SCRATCH_BYTES = 32 << 20
DTYPE_BF16, DTYPE_FP32 = 0, 1
OUTGOING, INCOMING = 0, 1
MASK_NONE, MASK_TOKEN, MASK_PAIR = 0, 1, 2
FLAG_PLAIN_KERNELS = 1
FLAG_SINGLE_CTA_CONTRACT = 2
FLAG_SINGLE_CTA_STAGE1 = 4
FLAG_INPLACE_NORM_STAGE3 = 16
FLAG_SERIAL_LAUNCH = 32

EXPORTED_SYMBOLS = (
    "trimul_b200_abi_version",
    "trimul_b200_strerror",
    "trimul_b200_workspace_bytes",
    "trimul_b200_forward",
    "trimul_b200_tm1",
    "trimul_b200_contract",
    "trimul_b200_tm2",
    "trimul_b200_forward_static",
    "trimul_b200_tm1_scatter",
    "trimul_b200_bidir_workspace_bytes",
    "trimul_b200_forward_bidir",
    "trimul_b200_contract_scatter",
    "trimul_b200_peer_barrier",
    "trimul_b200_selftest_expiring_wait",
)


class Desc(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32),
        ("B", C.c_int32), ("N", C.c_int32), ("c", C.c_int32), ("c_hidden", C.c_int32),
        ("dtype", C.c_int32), ("direction", C.c_int32), ("mask_kind", C.c_int32),
        ("eps_in", C.c_float), ("eps_out", C.c_float),
        ("flags", C.c_uint32),
        ("rows", C.c_int32), ("row0", C.c_int32),
        ("drop_scale", C.c_void_p),
    ]


class Weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "ln_in_weight", "ln_in_bias", "w_left", "w_left_gate", "w_right", "w_right_gate",
        "ln_out_weight", "ln_out_bias", "w_gate", "w_out")]


class Planes(C.Structure):
    _fields_ = [("base", C.c_void_p)] + [(n, C.c_int64) for n in (
        "rows", "cols", "pitch", "plane_stride", "chunk_stride", "row_chunk", "col_chunk")]


class TrimulLibraryError(RuntimeError):
    """The C-ABI library is missing, stale or returned an error code."""


_lib = None


def load():
    """Load the shared library once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TrimulLibraryError(
            f"{LIB_PATH} not found: build it with `python -m miniworld_engine_b200.build` "
            "(there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    lib.trimul_b200_abi_version.restype = C.c_int
    lib.trimul_b200_abi_version.argtypes = []
    lib.trimul_b200_strerror.restype = C.c_char_p
    lib.trimul_b200_strerror.argtypes = [C.c_int]
    PD, PW, PP = C.POINTER(Desc), C.POINTER(Weights), C.POINTER(Planes)
    lib.trimul_b200_workspace_bytes.restype = C.c_int
    lib.trimul_b200_workspace_bytes.argtypes = [PD, C.POINTER(C.c_size_t), PP, PP, PP]
    lib.trimul_b200_forward.restype = C.c_int
    lib.trimul_b200_forward.argtypes = [PD, C.c_void_p, C.c_void_p, PW, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.trimul_b200_tm1.restype = C.c_int
    lib.trimul_b200_tm1.argtypes = [PD, C.c_void_p, C.c_void_p, PW, PP, PP, C.c_void_p, C.c_void_p]
    lib.trimul_b200_contract.restype = C.c_int
    lib.trimul_b200_contract.argtypes = [C.c_int32, C.c_uint32, C.c_int32, PP, PP, PP, C.c_void_p, C.c_void_p]
    lib.trimul_b200_tm1_scatter.restype = C.c_int
    lib.trimul_b200_tm1_scatter.argtypes = [PD, C.c_void_p, C.c_void_p, PW, C.c_int32, PP, PP, C.c_void_p, C.c_void_p]
    lib.trimul_b200_contract_scatter.restype = C.c_int
    lib.trimul_b200_contract_scatter.argtypes = [C.c_int32, C.c_uint32, C.c_int32, PP, PP, C.c_int32, PP, C.c_void_p,
                                                 C.c_void_p]
    lib.trimul_b200_bidir_workspace_bytes.restype = C.c_int
    lib.trimul_b200_bidir_workspace_bytes.argtypes = [PD, C.POINTER(C.c_size_t)]
    lib.trimul_b200_forward_bidir.restype = C.c_int
    lib.trimul_b200_forward_bidir.argtypes = [PD, C.c_void_p, C.c_void_p, PW, C.c_void_p, C.c_int32, C.c_void_p,
                                              C.c_size_t, C.c_void_p, C.c_void_p]
    lib.trimul_b200_tm2.restype = C.c_int
    lib.trimul_b200_tm2.argtypes = [PD, C.c_void_p, PP, PW, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.trimul_b200_forward_static.restype = C.c_int
    lib.trimul_b200_forward_static.argtypes = [PD, C.c_void_p, C.c_void_p, PW, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.c_void_p]
    lib.trimul_b200_peer_barrier.restype = C.c_int
    lib.trimul_b200_peer_barrier.argtypes = [C.c_int32, C.c_int32, C.POINTER(C.c_void_p), C.c_uint32, C.c_uint32,
                                             C.c_void_p, C.c_void_p]
    lib.trimul_b200_selftest_expiring_wait.restype = C.c_int
    lib.trimul_b200_selftest_expiring_wait.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p]
    if lib.trimul_b200_abi_version() != ABI_VERSION:
        raise TrimulLibraryError(
            f"ABI mismatch: library {lib.trimul_b200_abi_version()}, binding {ABI_VERSION}; rebuild the library")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().trimul_b200_strerror(code).decode()


def check(code: int, what: str) -> None:
    """Turn a C-ABI return code into the exception the reference interface raises:
    ``NotImplementedError`` for unsupported configurations (as the reference's launchers do,
    ``kernels/tm1/cute/launch.py:239-240``), ``ValueError`` for invalid arguments,
    ``TrimulLibraryError`` for everything else."""
    if code == OK:
        return
    msg = f"{what}: {strerror(code)} (code {code})"
    if code == E_UNSUPPORTED:
        raise NotImplementedError(msg)
    if code == E_INVALID:
        raise ValueError(msg)
    raise TrimulLibraryError(msg)


def make_desc(B, N, c, *, dtype, direction, mask_kind=MASK_NONE, eps_in=1e-5, eps_out=1e-5,
              flags=0, rows=None, row0=0, c_hidden=None, drop_scale=None) -> Desc:
    """``drop_scale`` is a device address (``tensor.data_ptr()``) or None."""
    return Desc(C.sizeof(Desc), B, N, c, c if c_hidden is None else c_hidden, dtype, direction, mask_kind,
                eps_in, eps_out, flags, N if rows is None else rows, row0, drop_scale)
