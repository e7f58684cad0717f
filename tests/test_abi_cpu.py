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
    assert C.sizeof(_lib.Desc) == 64 and _lib.Desc.drop_scale.offset == 56     # 13 x 4 bytes, padding, one pointer
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


def test_parameter_struct_cache_is_keyed_by_what_the_struct_depends_on(monkeypatch):
    """The validated parameter struct is remembered under addresses, dtypes, shapes and contiguity:
    the same tensors hit it, a reshaped or transposed view of the same memory does not (and is
    validated afresh), and parameter sets that needed a conversion are never remembered."""
    import torch
    from miniworld_engine_b200 import functional as F
    monkeypatch.setattr(F, "_require_cuda", lambda t, name: None)      # CPU tensors stand in
    monkeypatch.setattr(F, "_struct_cache", {})
    c, h = 16, 8
    vec = lambda n: torch.ones(n)
    lin = lambda r, k: torch.zeros(r, k, dtype=torch.bfloat16)
    p = dict(ln_in_w=vec(c), ln_in_b=vec(c), w_left=lin(h, c), w_left_gate=lin(h, c), w_right=lin(h, c),
             w_right_gate=lin(h, c), ln_out_w=vec(h), ln_out_b=vec(h), w_gate=lin(c, c), w_out=lin(c, h))
    w1, k1 = F._weights_struct(c, torch.bfloat16, device=None, c_hidden=h, c_proj=h, **p)
    w2, k2 = F._weights_struct(c, torch.bfloat16, device=None, c_hidden=h, c_proj=h, **p)
    assert w1 is w2 and k1 == [] and k2 == [] and len(F._struct_cache) == 1
    assert w1.w_out == p["w_out"].data_ptr() and w1.ln_out_bias == p["ln_out_b"].data_ptr()
    # same memory seen as [h, c] instead of [c, h]: a different key, and the shape check fires
    with pytest.raises(ValueError, match="to_out.weight"):
        F._weights_struct(c, torch.bfloat16, device=None, c_hidden=h, c_proj=h, **{**p, "w_out": p["w_out"].view(h, c)})
    # a transposed (non-contiguous) square weight is converted to a copy, which is returned for
    # keeping alive and not remembered
    w3, k3 = F._weights_struct(c, torch.bfloat16, device=None, c_hidden=h, c_proj=h, **{**p, "w_gate": p["w_gate"].t()})
    assert len(k3) == 1 and w3.w_gate == k3[0].data_ptr() != p["w_gate"].data_ptr() and len(F._struct_cache) == 1
    # fp32 Linear weights for a bf16 call: converted, not remembered
    w4, k4 = F._weights_struct(c, torch.bfloat16, device=None, c_hidden=h, c_proj=h, **{**p, "w_left": p["w_left"].float()})
    assert len(k4) == 1 and k4[0].dtype == torch.bfloat16 and len(F._struct_cache) == 1
    # other expected widths with the same tensors: validated afresh and rejected
    with pytest.raises(ValueError):
        F._weights_struct(c, torch.bfloat16, device=None, c_hidden=c, c_proj=h, **p)


def test_functional_ops_refuse_to_detach_silently():
    """The functional entry points are forward-only: with grad enabled and an input or a parameter
    that requires grad they raise (the reference's op is autograd-transparent,
    kernels/trimul_inproj/whole_op.py:170-190), before any device check."""
    import torch
    from miniworld_engine_b200 import triangle_multiplicative_update_b200
    from miniworld_engine_b200.bidirectional import bidirectional_triangle_multiplicative_update_b200
    d = 16
    x = torch.zeros(1, 4, 4, d, requires_grad=True)
    v, m, m2 = torch.zeros(d), torch.zeros(d, d), torch.zeros(2 * d, d)
    with pytest.raises(NotImplementedError, match="forward-only"):
        triangle_multiplicative_update_b200(x, "outgoing", None, v, v, m2, m2, v, v, m, m)
    w = torch.zeros(2 * d, d, requires_grad=True)
    with pytest.raises(NotImplementedError, match="forward-only"):
        triangle_multiplicative_update_b200(x.detach(), "incoming", None, v, v, w, m2, v, v, m, m)
    v2, mo = torch.zeros(2 * d), torch.zeros(d, 2 * d)
    with pytest.raises(NotImplementedError, match="forward-only"):
        bidirectional_triangle_multiplicative_update_b200(
            x, None, norm_in_weight=v, norm_in_bias=v, to_left_weight=m2, to_left_gate_weight=m2,
            to_right_weight=m2, to_right_gate_weight=m2, norm_out_weight=v2, norm_out_bias=v2,
            to_out_weight=mo, to_gate_weight=m)
    # without grad the same calls get as far as the device check
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU path"):
        triangle_multiplicative_update_b200(x, "outgoing", None, v, v, m2, m2, v, v, m, m)


def test_descriptor_without_the_trailing_field_is_still_accepted(lib):
    """A caller built against the shorter descriptor (no drop_scale) passes its own struct_bytes."""
    from miniworld_engine_b200 import _lib
    d = _lib.make_desc(1, 16, 128, dtype=_lib.DTYPE_BF16, direction=_lib.OUTGOING)
    n_new, n_old = C.c_size_t(), C.c_size_t()
    assert lib.trimul_b200_workspace_bytes(C.byref(d), C.byref(n_new), None, None, None) == _lib.OK
    d.struct_bytes = 56
    d.drop_scale = 0xdead0                      # must be ignored: the short form has no such field
    assert lib.trimul_b200_workspace_bytes(C.byref(d), C.byref(n_old), None, None, None) == _lib.OK
    assert n_old.value == n_new.value
    d.struct_bytes = 60
    assert lib.trimul_b200_workspace_bytes(C.byref(d), C.byref(n_old), None, None, None) == _lib.E_INVALID


def test_barrier_and_selftest_argument_checks(lib):
    from miniworld_engine_b200 import _lib
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    assert lib.trimul_b200_peer_barrier(0, 9, ptrs, 1, 1000, None, None) == _lib.E_INVALID     # world > 8
    assert lib.trimul_b200_peer_barrier(2, 2, ptrs, 1, 1000, None, None) == _lib.E_INVALID     # rank outside
    assert lib.trimul_b200_peer_barrier(0, 2, ptrs, 0, 1000, None, None) == _lib.E_INVALID     # epoch 0
    assert lib.trimul_b200_peer_barrier(0, 2, ptrs, 1, 0, None, None) == _lib.E_INVALID        # no limit
    bad = (C.c_void_p * 2)(0x1000, None)
    assert lib.trimul_b200_peer_barrier(0, 2, bad, 1, 1000, None, None) == _lib.E_INVALID      # null flag array
    assert lib.trimul_b200_selftest_expiring_wait(1000, None, None) == _lib.E_INVALID          # status required
