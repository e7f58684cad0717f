"""The workspace-free entry point, ``trimul_b200_forward_static``.

It exists for hosts that cannot give the library a workspace: a server whose own pool owns
all device memory (a plugin's cudaMalloc would fail or take another tenant's budget), a
latency-critical loop that must avoid cudaMalloc's device-wide synchronisation, or a
foreign-function boundary that carries only inputs and outputs.  The scratch planes then live
in a fixed array inside the library's device image.

The test drives the entry point directly through the C ABI and compares it with the ordinary
``trimul_b200_forward`` (caller-supplied workspace) on two calls in a row — the second one
smaller and of the other direction, so it runs on top of whatever the first left in the
shared array.  This file sorts last on purpose: a run that stops at the first failure has
then already executed every other test.  It passes on its own in a fresh process too (the
first call on a device performs the one-time address look-up).
"""

import ctypes as C

import pytest
import torch

from oracle import trimul_oracle as O

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2     # same tolerance as tests/test_gpu_parity.py


def _weights_struct(w, dev, keep):
    from miniworld_engine_b200 import _lib
    wd = w.to(torch.bfloat16)

    def p(t, dt):
        t = t.to(dev).to(dt).contiguous()
        keep.append(t)
        return t.data_ptr()

    return _lib.Weights(
        p(wd.ln_pair_weight, torch.float32), p(wd.ln_pair_bias, torch.float32),
        p(wd.to_left, torch.bfloat16), p(wd.to_left_gate, torch.bfloat16),
        p(wd.to_right, torch.bfloat16), p(wd.to_right_gate, torch.bfloat16),
        p(wd.ln_out_weight, torch.float32), p(wd.ln_out_bias, torch.float32),
        p(wd.to_gate, torch.bfloat16), p(wd.to_out, torch.bfloat16))


def _both_entry_points(N, outgoing, mask_kind, seed, dev):
    """Run the same problem through the static-scratch entry point and through the ordinary
    one; returns (static result, ordinary result, oracle result) on the CPU."""
    from miniworld_engine_b200 import _lib
    lib = _lib.load()
    keep = []
    w = O.make_weights(128, seed, affine="random")
    z = O.make_input(1, N, 128, seed + 1).bfloat16()
    m = O.make_token_mask(1, N, mask_kind)
    zd, md = z.to(dev), m.to(dev).view(torch.uint8)
    ws = _weights_struct(w, dev, keep)
    desc = _lib.make_desc(1, N, 128, dtype=_lib.DTYPE_BF16,
                          direction=_lib.OUTGOING if outgoing else _lib.INCOMING, mask_kind=_lib.MASK_TOKEN)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    out_static = torch.empty_like(zd)
    rc = lib.trimul_b200_forward_static(C.byref(desc), zd.data_ptr(), md.data_ptr(), C.byref(ws),
                                        out_static.data_ptr(), None, stream, status.data_ptr())
    assert rc == 0, _lib.strerror(rc)

    need = C.c_size_t()
    assert lib.trimul_b200_workspace_bytes(C.byref(desc), C.byref(need), None, None, None) == 0
    assert need.value <= _lib.STATIC_SCRATCH_BYTES
    workspace = torch.empty(need.value, dtype=torch.uint8, device=dev)
    out_plain = torch.empty_like(zd)
    rc = lib.trimul_b200_forward(C.byref(desc), zd.data_ptr(), md.data_ptr(), C.byref(ws),
                                 out_plain.data_ptr(), None, workspace.data_ptr(), need.value, stream,
                                 status.data_ptr())
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize(dev)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    ref = O.trimul_forward(z, m, w.to(torch.bfloat16), outgoing)
    return out_static.cpu(), out_plain.cpu(), ref


def test_static_scratch_entry_point_matches_workspace_entry_point():
    dev = torch.device("cuda", 0)
    with torch.cuda.device(dev):
        # two calls in a row on the shared array: a larger outgoing problem, then a smaller
        # incoming one that only partly overwrites what the first left behind
        for N, outgoing, mask_kind, seed in ((160, True, "tail11", 40), (61, False, "tail5", 50)):
            got, want, ref = _both_entry_points(N, outgoing, mask_kind, seed, dev)
            assert not torch.isnan(got.float()).any()
            err = O.rel_rms(got.float(), want.float())
            assert err <= TOL_BF16, f"N={N}: static vs workspace entry point rel-RMS {err:.3e}"
            assert torch.equal(got, want), "same kernels on the same layout should agree bit for bit"
            err_ref = O.rel_rms(got.float(), ref.float())
            assert err_ref <= TOL_BF16, f"N={N}: static entry point vs oracle rel-RMS {err_ref:.3e}"


def test_static_scratch_entry_point_refuses_oversized_problems():
    from miniworld_engine_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    with torch.cuda.device(dev):
        desc = _lib.make_desc(1, 512, 128, dtype=_lib.DTYPE_BF16, direction=_lib.OUTGOING)
        need = C.c_size_t()
        assert lib.trimul_b200_workspace_bytes(C.byref(desc), C.byref(need), None, None, None) == 0
        assert need.value > _lib.STATIC_SCRATCH_BYTES
        x = torch.zeros(1, 512, 512, 128, dtype=torch.bfloat16, device=dev)
        y = torch.empty_like(x)
        keep = []
        ws = _weights_struct(O.make_weights(128, 0), dev, keep)
        rc = lib.trimul_b200_forward_static(C.byref(desc), x.data_ptr(), None, C.byref(ws), y.data_ptr(), None,
                                            torch.cuda.current_stream(dev).cuda_stream, None)
        assert rc == _lib.E_STATIC_SCRATCH
        assert "built-in" in _lib.strerror(rc)
