"""CPU-only checks of the C ABI: the library builds, loads and exports every symbol the header
declares; argument validation works without a GPU (no compute call is made)."""

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from miniworld_engine_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "trimul_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trimul_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    from miniworld_engine_b200 import _lib
    names = declared_functions()
    assert len(names) >= 7
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/trimul_b200.h but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) <= set(names)


def test_struct_layouts_match_header(lib):
    from miniworld_engine_b200 import _lib
    assert C.sizeof(_lib.Desc) == 13 * 4
    assert C.sizeof(_lib.Weights) == 10 * 8
    assert C.sizeof(_lib.Planes) == 8 * 8
    assert lib.trimul_b200_abi_version() == _lib.ABI_VERSION


def test_strerror_covers_all_codes(lib):
    from miniworld_engine_b200 import _lib
    for code in (0, -1, -2, -3, -4, -5):
        assert _lib.strerror(code) and "unknown" not in _lib.strerror(code)
    assert "unknown" in _lib.strerror(-99)


def test_workspace_layout(lib):
    from miniworld_engine_b200 import _lib
    d = _lib.make_desc(2, 61, 128, dtype=_lib.DTYPE_BF16, direction=_lib.INCOMING)
    n, a, b, t = C.c_size_t(), _lib.Planes(), _lib.Planes(), _lib.Planes()
    assert lib.trimul_b200_workspace_bytes(C.byref(d), C.byref(n), C.byref(a), C.byref(b), C.byref(t)) == 0
    assert a.pitch == 64 and a.rows == 61 and a.cols == 61 and a.plane_stride == 61 * 64
    assert (a.base or 0) == 0 and b.base % 1024 == 0 and t.base == 2 * b.base
    assert n.value >= 3 * 2 * 128 * 61 * 64 * 2


def test_validation_without_gpu(lib):
    from miniworld_engine_b200 import _lib
    n = C.c_size_t()
    bad = _lib.make_desc(1, 0, 128, dtype=0, direction=0)
    assert lib.trimul_b200_workspace_bytes(C.byref(bad), C.byref(n), None, None, None) == _lib.E_INVALID
    bad = _lib.make_desc(1, 8, 128, dtype=7, direction=0)
    assert lib.trimul_b200_workspace_bytes(C.byref(bad), C.byref(n), None, None, None) == _lib.E_INVALID
    bad = _lib.make_desc(1, 8, 128, dtype=0, direction=0, c_hidden=60)
    assert lib.trimul_b200_workspace_bytes(C.byref(bad), C.byref(n), None, None, None) == _lib.E_UNSUPPORTED
    bad = _lib.make_desc(1, 8, 128, dtype=0, direction=0, c_hidden=264)
    assert lib.trimul_b200_workspace_bytes(C.byref(bad), C.byref(n), None, None, None) == _lib.E_UNSUPPORTED
    # d_hidden != d_pair: the scratch holds B * c_hidden planes per operand
    half = _lib.make_desc(1, 8, 128, dtype=0, direction=0, c_hidden=64)
    full = _lib.make_desc(1, 8, 128, dtype=0, direction=0)
    n_half, n_full = C.c_size_t(), C.c_size_t()
    assert lib.trimul_b200_workspace_bytes(C.byref(half), C.byref(n_half), None, None, None) == _lib.OK
    assert lib.trimul_b200_workspace_bytes(C.byref(full), C.byref(n_full), None, None, None) == _lib.OK
    assert 0 < n_half.value < n_full.value
    # the bidirectional block takes c_hidden = 2h, h a multiple of 8
    assert lib.trimul_b200_bidir_workspace_bytes(C.byref(_lib.make_desc(1, 8, 128, dtype=0, direction=0, c_hidden=128)),
                                                 C.byref(n)) == _lib.OK
    assert lib.trimul_b200_bidir_workspace_bytes(C.byref(_lib.make_desc(1, 8, 128, dtype=0, direction=0, c_hidden=72)),
                                                 C.byref(n)) == _lib.E_INVALID
    bad = _lib.make_desc(1, 8, 100, dtype=0, direction=0)
    assert lib.trimul_b200_workspace_bytes(C.byref(bad), C.byref(n), None, None, None) == _lib.E_UNSUPPORTED
    ok = _lib.make_desc(1, 8, 128, dtype=0, direction=0)
    # forward with null buffers is rejected before anything touches a device
    rc = lib.trimul_b200_forward(C.byref(ok), None, None, None, None, None, None, 0, None, None)
    assert rc == _lib.E_INVALID


def test_python_mirror_fails_loudly_on_cpu_tensors():
    import torch
    from miniworld_engine_b200 import TriangleMultiplicationB200
    mod = TriangleMultiplicationB200(128).eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU path"):
        mod(torch.zeros(1, 4, 4, 128))


def test_module_mirrors_reference_parameters():
    import torch
    from miniworld_engine_b200 import TriangleMultiplicationB200
    from oracle import trimul_oracle as O
    mod = TriangleMultiplicationB200(64, outgoing=False)
    w = O.make_weights(64, 3, affine="random")
    assert set(mod.state_dict().keys()) == set(w.state_dict().keys())
    mod.load_state_dict(w.state_dict())
    mod = mod.to(torch.bfloat16)
    wb = w.to(torch.bfloat16)
    # LayerNorm parameters stay fp32 tensors but carry bf16-rounded values, like the reference
    assert mod.ln_pair.weight.dtype == torch.float32
    assert torch.equal(mod.ln_pair.weight.data, wb.ln_pair_weight)
    assert mod.to_out.weight.dtype == torch.bfloat16 and torch.equal(mod.to_out.weight.data, wb.to_out)
    with pytest.raises(ValueError):
        TriangleMultiplicationB200(64, d_hidden=32)


def test_functional_op_reads_d_hidden_off_the_packed_projections():
    """Argument checks that need no device: an odd leading dimension of p_in_weight and a width
    mismatch raise ValueError (whole_op.py:203-207); a consistent d_hidden != d_pair passes them
    and then fails loudly on the CPU tensor."""
    import torch
    from miniworld_engine_b200 import triangle_multiplicative_update_b200 as f
    d, h = 32, 16
    x = torch.zeros(1, 4, 4, d)
    v_d, v_h = torch.ones(d), torch.ones(h)
    p_in, p_out, g_out = torch.zeros(2 * h, d), torch.zeros(d, h), torch.zeros(d, d)
    with pytest.raises(ValueError, match="even"):
        f(x, "outgoing", None, v_d, v_d, p_in[:-1], p_in[:-1], v_h, v_h, p_out, g_out)
    with pytest.raises(ValueError):
        f(x, "outgoing", None, v_d, v_d, p_in, torch.zeros(2 * h, d + 8), v_h, v_h, p_out, g_out)
    with pytest.raises(RuntimeError, match="no CPU path"):
        f(x, "outgoing", None, v_d, v_d, p_in, p_in, v_h, v_h, p_out, g_out)
