"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the
golden fixtures generated from the reference.

Tolerances (relative RMS error, ``||y - ref|| / ||ref||``):
  * fp32 path  <= 1e-5 against the fp32 oracle / fixture
  * bf16 path  <= 1e-2 against the bf16 oracle / fixture
"""

import glob
import os

import pytest
import torch

from oracle import trimul_oracle as O
from tests._util import forward_kwargs, oracle_out
from tests.test_oracle_golden import FILES, load_case, load_drop_scale

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5
TOL_BF16 = 1e-2


@pytest.fixture(scope="module")
def dev():
    import miniworld_engine_b200  # noqa: F401  (fails loudly if the package is broken)
    from miniworld_engine_b200 import _lib
    _lib.load()
    return torch.device("cuda", 0)


def run_block(z, mask, w, outgoing, dtype, dev, **kw):
    from miniworld_engine_b200 import read_status, trimul_forward
    y = trimul_forward(z.to(dtype).to(dev), None if mask is None else mask.to(dev), outgoing=outgoing,
                       **forward_kwargs(w, dtype, dev), **kw)
    st = read_status(dev)
    assert st[0] == 0, f"device status {st}"
    return y.cpu()


def run_bidir(z, mask, w, dtype, dev, **kw):
    """The bidirectional block (residual included, as the reference module returns it)."""
    from miniworld_engine_b200 import bidir_trimul_forward, read_status
    wd = w.to(dtype)
    t = lambda x: x.to(dev)
    y = bidir_trimul_forward(
        z.to(dtype).to(dev), None if mask is None else mask.to(dev),
        ln_in_weight=t(wd.ln_pair_weight), ln_in_bias=t(wd.ln_pair_bias), w_left=t(wd.to_left),
        w_left_gate=t(wd.to_left_gate), w_right=t(wd.to_right), w_right_gate=t(wd.to_right_gate),
        ln_out_weight=t(wd.ln_out_weight), ln_out_bias=t(wd.ln_out_bias), w_gate=t(wd.to_gate), w_out=t(wd.to_out),
        eps_in=w.eps_in, eps_out=w.eps_out, **kw)
    st = read_status(dev)
    assert st[0] == 0, f"device status {st}"
    return y.cpu()


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f)[:-4] for f in FILES])
def test_golden_fixture(path, dev):
    name, z, mask, w, gold, dtype, direction, form = load_case(path)
    if form == "module":
        y = run_block(z, mask, w, direction == "outgoing", dtype, dev)
    elif form == "bidir":
        y = run_bidir(z, mask, w, dtype, dev)
    elif form == "dropout":
        # what the reference module returns in training mode: block * scale + pair, in one call
        zd = z.to(dtype).to(dev)
        ds = load_drop_scale(path, dtype).to(dev)
        from miniworld_engine_b200 import read_status, trimul_forward
        y = trimul_forward(zd, None if mask is None else mask.to(dev), outgoing=(direction == "outgoing"),
                           **forward_kwargs(w, dtype, dev), residual=zd, drop_scale=ds).cpu()
        assert read_status(dev)[0] == 0
    else:
        from miniworld_engine_b200 import triangle_multiplicative_update_b200 as f
        wd = w.to(dtype)
        y = f(z.to(dtype).to(dev), direction, mask.to(dev),
              wd.ln_pair_weight.to(dev), wd.ln_pair_bias.to(dev),
              torch.cat([wd.to_left, wd.to_right]).to(dev), torch.cat([wd.to_left_gate, wd.to_right_gate]).to(dev),
              wd.ln_out_weight.to(dev), wd.ln_out_bias.to(dev), wd.to_out.to(dev), wd.to_gate.to(dev), 1e-5).cpu()
    assert y.dtype == dtype and tuple(y.shape) == tuple(gold.shape)
    err = O.rel_rms(y.float(), gold)
    tol = TOL_FP32 if dtype == torch.float32 else TOL_BF16
    assert err <= tol, f"{name}: rel-RMS {err:.3e} > {tol}"


def test_cfg1_outgoing_fp32_n32(dev):
    w, z, m = O.make_weights(128, 0), O.make_input(1, 32, 128, 1), O.make_token_mask(1, 32, "ones")
    y = run_block(z, m, w, True, torch.float32, dev)
    err = O.rel_rms(y, O.trimul_forward(z, m, w, True))
    assert err <= TOL_FP32, f"rel-RMS {err:.3e}"


@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
@pytest.mark.parametrize("N,B,mask_kind,affine", [
    (32, 1, "ones", "unit"),
    (61, 1, "tail7", "random"),
    (128, 2, "rand5", "random"),
    (129, 1, "tail20", "random"),
    (200, 1, None, "unit"),
    (384, 1, "ones", "unit"),          # BASELINE config 2 (outgoing)
])
def test_bf16_c128_block_vs_oracle(N, B, mask_kind, affine, outgoing, dev):
    w = O.make_weights(128, 0, affine=affine)
    z = O.make_input(B, N, 128, 1)
    m = None if mask_kind is None else O.make_token_mask(B, N, mask_kind)
    y = run_block(z, m, w, outgoing, torch.bfloat16, dev)
    ref16 = oracle_out(z, m, w, outgoing, torch.bfloat16)
    ref32 = O.trimul_forward(z.bfloat16().float(), m, w.to(torch.bfloat16).to(torch.float32), outgoing)
    e16, e32 = O.rel_rms(y.float(), ref16.float()), O.rel_rms(y.float(), ref32)
    print(f"N={N} B={B} {'out' if outgoing else 'in'}: vs bf16 oracle {e16:.3e}, vs fp32 oracle {e32:.3e}")
    assert e16 <= TOL_BF16 and e32 <= TOL_BF16


def test_cfg3_incoming_bf16_n768_tail77(dev):
    w, z, m = O.make_weights(128, 0), O.make_input(1, 768, 128, 1), O.make_token_mask(1, 768, "tail77")
    y = run_block(z, m, w, False, torch.bfloat16, dev)
    ref = oracle_out(z, m, w, False, torch.bfloat16)
    err = O.rel_rms(y.float(), ref.float())
    assert err <= TOL_BF16, f"rel-RMS {err:.3e}"
    # padded rows/columns of a, b are exactly zero, so with beta_out = 0 the padded outputs
    # equal sigmoid(.) * (Wo . 0) = 0 in the reference and here alike
    assert float(y[:, 768 - 77:, 768 - 77:].float().abs().max()) == float(ref[:, 768 - 77:, 768 - 77:].float().abs().max())


@pytest.mark.parametrize("c", [64, 128, 256])
def test_cfg4_outgoing_bf16_b2_n512_dpair_sweep(c, dev):
    w, z = O.make_weights(c, 0), O.make_input(2, 512, c, 1)
    m = O.make_token_mask(2, 512, "ones")
    y = run_block(z, m, w, True, torch.bfloat16, dev)
    err = O.rel_rms(y.float(), oracle_out(z, m, w, True, torch.bfloat16).float())
    assert err <= TOL_BF16, f"c={c}: rel-RMS {err:.3e}"


@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
@pytest.mark.parametrize("c,B,N,mask_kind", [
    (64, 2, 70, "tail7"), (256, 1, 65, "rand5"), (48, 1, 33, None), (32, 1, 130, "tail20"), (208, 1, 20, "tail3"),
], ids=["c64", "c256", "c48", "c32", "c208"])
def test_bf16_other_widths_take_the_warp_mma_kernels(dev, c, B, N, mask_kind, outgoing):
    """bf16 with c != 128 (a multiple of 16): stages 1 and 3 run on the warp-MMA kernels.  Checked
    against the oracle and, stage by stage on a row slab (rows < N, row0 > 0), against the scalar
    CUDA-core kernels, which round at the same points."""
    from miniworld_engine_b200 import stages as S
    from tests._util import weights_dict
    w = O.make_weights(c, 5, affine="random")
    z = O.make_input(B, N, c, 6)
    m = None if mask_kind is None else O.make_token_mask(B, N, mask_kind)
    y = run_block(z, m, w, outgoing, torch.bfloat16, dev)
    ref = oracle_out(z, m, w, outgoing, torch.bfloat16)
    err = O.rel_rms(y.float(), ref.float())
    assert err <= TOL_BF16, f"rel-RMS {err:.3e}"
    y_plain = run_block(z, m, w, outgoing, torch.bfloat16, dev, plain_kernels=True)
    assert O.rel_rms(y.float(), y_plain.float()) <= TOL_BF16
    # stage 1 and stage 3 on a slab of rows
    row0, rows = N // 3, N - N // 3 - 2
    zs = z.bfloat16().to(dev)[:, row0:row0 + rows].contiguous()
    md = None if m is None else m.to(dev)
    wd = weights_dict(w, torch.bfloat16, dev)
    pr, pc = (rows, N) if outgoing else (N, rows)
    got, want = [], []
    for plain, dst in ((False, got), (True, want)):
        a = S.alloc_planes(B * c, pr, pc, torch.bfloat16, dev, fill=0)
        b = S.alloc_planes(B * c, pr, pc, torch.bfloat16, dev, fill=0)
        S.tm1(zs, md, wd, a, b, outgoing=outgoing, row0=row0, plain_kernels=plain)
        dst += [S.planes_to_dense(a).float().cpu(), S.planes_to_dense(b).float().cpu()]
    for g, wnt in zip(got, want):
        assert O.rel_rms(g, wnt) <= 4e-3            # same rounding points, different summation order
        assert torch.equal(g == 0, wnt == 0)        # the masked positions are exactly zero in both
    tri = S.alloc_planes(B * c, rows, N, torch.bfloat16, dev)
    tri.buf.copy_(torch.randn(tri.buf.shape, generator=torch.Generator().manual_seed(9)).bfloat16())
    o1 = S.tm2(zs, tri, wd, residual=zs, row0=row0).float().cpu()
    o2 = S.tm2(zs, tri, wd, residual=zs, row0=row0, plain_kernels=True).float().cpu()
    assert O.rel_rms(o1 - zs.float().cpu(), o2 - zs.float().cpu()) <= 2e-2      # the update alone; both round the sum to bf16


def test_pair_mask_and_token_mask_agree(dev):
    w, z = O.make_weights(128, 5, affine="random"), O.make_input(1, 96, 128, 6)
    m = O.make_token_mask(1, 96, "rand5", seed=9)
    pm = m.unsqueeze(-1) & m.unsqueeze(-2)
    for outgoing in (True, False):
        a = run_block(z, m, w, outgoing, torch.bfloat16, dev)
        b = run_block(z, pm, w, outgoing, torch.bfloat16, dev)
        assert torch.equal(a, b)


def test_mask_none_equals_all_ones_and_batches_are_independent(dev):
    w, z = O.make_weights(128, 0), O.make_input(2, 160, 128, 1)
    ones = O.make_token_mask(2, 160, "ones")
    a = run_block(z, None, w, True, torch.bfloat16, dev)
    b = run_block(z, ones, w, True, torch.bfloat16, dev)
    assert torch.equal(a, b)
    c1 = run_block(z[1:2], None, w, True, torch.bfloat16, dev)
    assert torch.equal(a[1:2], c1)


def test_residual_matches_reference_module_semantics(dev):
    """out + pair is a bf16 add of the bf16-rounded block output (module.py:453).  The residual
    that IS the input takes the default last stage (it adds the z tile it already holds); any
    other residual tensor takes the in-place-normalising variant, which has a tile buffer for it."""
    from miniworld_engine_b200 import read_status, trimul_forward
    w, z = O.make_weights(128, 0), O.make_input(1, 130, 128, 1)
    kw = forward_kwargs(w, torch.bfloat16, dev)
    zd = z.bfloat16().to(dev)
    other = O.make_input(1, 130, 128, 7).bfloat16().to(dev)
    y = trimul_forward(zd, None, outgoing=True, **kw)
    yr = trimul_forward(zd, None, outgoing=True, residual=zd, **kw)
    assert torch.equal(yr, y + zd)
    y_inplace = trimul_forward(zd, None, outgoing=True, inplace_norm=True, **kw)
    yo = trimul_forward(zd, None, outgoing=True, residual=other, **kw)
    assert torch.equal(yo, y_inplace + other)
    yz = trimul_forward(zd, None, outgoing=True, residual=zd.clone(), **kw)
    assert torch.equal(yz, y_inplace + zd)
    assert read_status(dev)[0] == 0


def test_tensor_core_kernels_match_plain_kernels(dev):
    """Same layouts, same rounding points: the tcgen05 path and the CUDA-core path agree to
    within a few bf16 ulps of accumulated difference."""
    w, z = O.make_weights(128, 0, affine="random"), O.make_input(1, 192, 128, 1)
    m = O.make_token_mask(1, 192, "tail13")
    for outgoing in (True, False):
        fast = run_block(z, m, w, outgoing, torch.bfloat16, dev)
        plain = run_block(z, m, w, outgoing, torch.bfloat16, dev, plain_kernels=True)
        err = O.rel_rms(fast.float(), plain.float())
        assert err <= 4e-3, f"rel-RMS {err:.3e}"


def test_poisoned_workspace_gives_identical_result(dev):
    """Nothing may depend on what the scratch planes held before the call (pitch padding,
    out-of-range tile parts): NaN-filling the workspace must not change a single bit."""
    from miniworld_engine_b200 import functional as Fn
    w, z = O.make_weights(128, 0), O.make_input(1, 77, 128, 1)
    m = O.make_token_mask(1, 77, "tail9")
    a = run_block(z, m, w, False, torch.bfloat16, dev)
    for buf in Fn._workspaces.values():
        buf.view(torch.int16).fill_(0x7FC0)      # bf16 NaN pattern
    b = run_block(z, m, w, False, torch.bfloat16, dev)
    assert torch.equal(a, b) and not torch.isnan(b.float()).any()


def test_errors_follow_the_reference_interface(dev):
    from miniworld_engine_b200 import TriangleMultiplicationB200, triangle_multiplicative_update_b200 as f
    x = torch.zeros(1, 8, 8, 128, device=dev, dtype=torch.bfloat16)
    v, W2, W1 = torch.ones(128, device=dev), torch.zeros(256, 128, device=dev), torch.zeros(128, 128, device=dev)
    with pytest.raises(ValueError):
        f(x, "sideways", None, v, v, W2, W2, v, v, W1, W1)
    with pytest.raises(ValueError):
        TriangleMultiplicationB200(128, d_hidden=64)
    with pytest.raises(NotImplementedError):
        f(x.half(), "outgoing", None, v, v, W2, W2, v, v, W1, W1)
    with pytest.raises(RuntimeError):
        f(x.cpu(), "outgoing", None, v, v, W2, W2, v, v, W1, W1)


def test_module_state_dict_roundtrip_and_forward(dev):
    from miniworld_engine_b200 import TriangleMultiplicationB200
    w = O.make_weights(128, 0, affine="random")
    mod = TriangleMultiplicationB200(128, outgoing=False)
    mod.load_state_dict(w.state_dict())
    mod = mod.to(dev).to(torch.bfloat16).eval()
    assert mod.ln_pair.weight.dtype == torch.float32 and mod.to_left.weight.dtype == torch.bfloat16
    z = O.make_input(1, 64, 128, 1).bfloat16()
    m = O.make_token_mask(1, 64, "tail5")
    with torch.no_grad():
        y = mod(z.to(dev), m.to(dev)).cpu()
    ref = O.trimul_forward(z, m, w.to(torch.bfloat16), False) + z
    assert O.rel_rms(y.float(), ref.float()) <= TOL_BF16


def test_alternative_kernels_agree(dev):
    """The lone-CTA contraction is another schedule of the same arithmetic as the CTA-pair one
    (same accumulation order per output element): bit-identical.  The lone-CTA stage 1 is another split of the same arithmetic as the CTA-pair one (same
    LayerNorm summation order, same K order in the projections): bit-identical too."""
    from miniworld_engine_b200 import read_status, stages as S
    from tests._util import weights_dict
    w = O.make_weights(128, 0, affine="random")
    wd = weights_dict(w, torch.bfloat16, dev)
    N = 200
    z = O.make_input(2, N, 128, 1).bfloat16().to(dev)
    m = O.make_token_mask(2, N, "tail9").to(dev)
    for outgoing in (True, False):
        res = []
        for single_cta in (False, True):
            a = S.alloc_planes(256, N, N, torch.bfloat16, dev, fill=float("nan"))
            b = S.alloc_planes(256, N, N, torch.bfloat16, dev, fill=float("nan"))
            S.tm1(z, m, wd, a, b, outgoing=outgoing, single_cta=single_cta)
            res.append((S.planes_to_dense(a).clone(), S.planes_to_dense(b).clone(), a, b))
        assert torch.equal(res[1][0], res[0][0]) and torch.equal(res[1][1], res[0][1])
        assert bool((res[0][0] == 0).any())                     # masked positions: exact zeros
        t1 = S.alloc_planes(256, N, N, torch.bfloat16, dev, fill=float("nan"))
        t2 = S.alloc_planes(256, N, N, torch.bfloat16, dev, fill=float("nan"))
        S.contract(res[0][2], res[0][3], t1)
        S.contract(res[0][2], res[0][3], t2, single_cta=True)
        assert torch.equal(S.planes_to_dense(t1), S.planes_to_dense(t2))
        # stage 3: default (both LayerNorms folded into the weights) against the in-place variant,
        # with and without the residual
        for residual in (None, z):
            y_fold = S.tm2(z, t1, wd, residual=residual)
            y_inpl = S.tm2(z, t1, wd, residual=residual, inplace_norm=True)
            assert O.rel_rms(y_fold.float().cpu(), y_inpl.float().cpu()) <= 6e-3
    assert read_status(dev)[0] == 0


def test_folded_norm_is_no_further_from_fp32_than_the_reference_bf16_path(dev):
    """The default stage 3 rounds W*gamma to bf16 where the reference rounds LN(x).  Neither is
    'the' answer; measured against an fp32 evaluation of the same bf16 inputs the folded form must
    not be worse than the reference's own bf16 path (plus a little slack)."""
    from miniworld_engine_b200 import trimul_forward
    from tests._util import forward_kwargs
    for affine, shift in (("unit", 0.0), ("random", 0.0), ("random", 4.0)):
        w = O.make_weights(128, 3, affine=affine)
        z = (O.make_input(1, 192, 128, 5) + shift).bfloat16()
        wb = w.to(torch.bfloat16)
        truth = O.trimul_forward(z.float(), None, wb.to(torch.float32), True)
        ref_bf16 = O.trimul_forward(z, None, wb, True).float()
        y = trimul_forward(z.to(dev), None, outgoing=True, **forward_kwargs(w, torch.bfloat16, dev)).float().cpu()
        e_ref, e_ours = O.rel_rms(ref_bf16, truth), O.rel_rms(y, truth)
        assert e_ours <= 1.1 * e_ref, f"{affine}, shift {shift}: ours {e_ours:.3e} vs reference bf16 {e_ref:.3e}"


def test_cuda_graph_capture_and_replay(dev):
    """The block call neither allocates nor synchronises once its buffers exist, so it can be
    captured in a CUDA graph; replays must reproduce the eager result bit for bit (the reference
    benchmarks its own path in this regime, benchmarks/runners/bench.py:295-344)."""
    from miniworld_engine_b200 import read_status, stages as S
    from tests._util import weights_dict
    w = O.make_weights(128, 0)
    wd = weights_dict(w, torch.bfloat16, dev)
    N = 160
    z = O.make_input(1, N, 128, 1).bfloat16().to(dev)
    m = O.make_token_mask(1, N, "tail7").to(dev)
    a = S.alloc_planes(128, N, N, torch.bfloat16, dev)
    b = S.alloc_planes(128, N, N, torch.bfloat16, dev)
    t = S.alloc_planes(128, N, N, torch.bfloat16, dev)

    def block():
        S.tm1(z, m, wd, a, b, outgoing=False)
        S.contract(a, b, t)
        return S.tm2(z, t, wd, residual=z)

    eager = block().clone()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        block()                                   # warm-up on the capture stream (module load, attributes)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = block()
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize(dev)
        assert torch.equal(out, eager)
    assert read_status(dev)[0] == 0


@pytest.mark.parametrize("B,N,mask_kind,affine", [(1, 128, "ones", "unit"), (1, 200, "tail9", "random"),
                                                  (2, 96, "rand5", "random")])
def test_bidirectional_block_bf16_tensor_core_path(dev, B, N, mask_kind, affine):
    """d = h = 128, bf16: stage 1 twice (one direction each), one contraction over 256 planes per
    batch element, the wide last stage (LayerNorm over 256 channels folded into a [128, 256]
    projection).  Oracle: the eager branch of the reference's bidirectional module."""
    w = O.make_bidir_weights(128, 128, 7, affine=affine)
    z = O.make_input(B, N, 128, 8)
    m = O.make_token_mask(B, N, mask_kind, seed=9)
    ref = O.bidir_forward(z.bfloat16(), m, w.to(torch.bfloat16)).float()
    y = run_bidir(z, m, w, torch.bfloat16, dev).float()
    err = O.rel_rms(y, ref)
    assert err <= TOL_BF16, f"rel-RMS {err:.3e}"
    # the block's own contribution (without the residual that dominates the norm) must agree too
    zb = z.bfloat16().float()
    e_upd = O.rel_rms(y - zb, ref - zb)
    assert e_upd <= 2e-2, f"update-only rel-RMS {e_upd:.3e}"
    # tensor-core kernels against the CUDA-core kernels of the same library
    y_plain = run_bidir(z, m, w, torch.bfloat16, dev, plain_kernels=True).float()
    assert O.rel_rms(y - zb, y_plain - zb) <= 1.5e-2
    # without the residual
    y_nores = run_bidir(z, m, w, torch.bfloat16, dev, add_residual=False).float()
    ref_nores = O.bidir_forward(z.bfloat16(), m, w.to(torch.bfloat16), add_residual=False).float()
    assert O.rel_rms(y_nores, ref_nores) <= TOL_BF16


def test_bidirectional_block_fp32(dev):
    w = O.make_bidir_weights(64, 64, 3, affine="random")
    z = O.make_input(2, 40, 64, 4)
    m = O.make_token_mask(2, 40, "tail5")
    y = run_bidir(z, m, w, torch.float32, dev)
    err = O.rel_rms(y, O.bidir_forward(z, m, w))
    assert err <= TOL_FP32, f"rel-RMS {err:.3e}"


@pytest.mark.parametrize("dtype,d,h,B,N,mask_kind", [
    (torch.float32, 32, 16, 2, 21, "tail3"),
    (torch.float32, 64, 128, 1, 18, None),
    (torch.bfloat16, 128, 64, 1, 150, "rand5"),     # CUDA-core stage 1, tensor-core contraction and stage 3
    (torch.bfloat16, 64, 32, 2, 37, "tail5"),
    (torch.bfloat16, 128, 96, 1, 40, "tail4"),      # 2h = 192: CUDA-core stage 3 as well
], ids=["fp32_d32_h16", "fp32_d64_h128", "bf16_d128_h64", "bf16_d64_h32", "bf16_d128_h96"])
def test_bidirectional_block_with_d_hidden_unequal_d_pair(dev, dtype, d, h, B, N, mask_kind):
    """``BidirectionalTriangleMultiplication(d_pair, d_hidden)`` with ``d_hidden != d_pair``
    (bidirectional.py:73-84): projections [2h, d], LayerNorm_out over 2h, to_out [d, 2h]."""
    w = O.make_bidir_weights(d, h, 61, affine="random")
    z = O.make_input(B, N, d, 62)
    m = None if mask_kind is None else O.make_token_mask(B, N, mask_kind)
    y = run_bidir(z, m, w, dtype, dev).float()
    ref = O.bidir_forward(z.to(dtype), m, w.to(dtype)).float()
    zb = z.to(dtype).float()
    if dtype == torch.float32:
        assert O.rel_rms(y, ref) <= TOL_FP32
        assert O.rel_rms(y - zb, ref - zb) <= 2e-5
    else:
        assert O.rel_rms(y, ref) <= TOL_BF16
        assert O.rel_rms(y - zb, ref - zb) <= 2e-2      # the update alone, without the dominating residual


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("dtype,d,h,B,N", [
    (torch.float32, 32, 16, 2, 19),
    (torch.float32, 32, 64, 1, 17),
    (torch.bfloat16, 128, 64, 1, 130),
    (torch.bfloat16, 128, 256, 1, 72),      # tensor-core contraction and (2 x 128-channel) stage 3
    (torch.bfloat16, 64, 32, 2, 33),
], ids=["fp32_d32_h16", "fp32_d32_h64", "bf16_d128_h64", "bf16_d128_h256", "bf16_d64_h32"])
def test_functional_op_with_d_hidden_unequal_d_pair(dev, dtype, d, h, B, N, direction):
    """The functional op reads d_hidden off the packed projections, p_in / g_in [2h, d], norm_out (h,),
    p_out [d, h] (whole_op.py:170-209); pair mask [B, L, L]."""
    from miniworld_engine_b200 import read_status, triangle_multiplicative_update_b200 as f
    w = O.make_weights(d, 71, affine="random", h=h).to(dtype)
    z = O.make_input(B, N, d, 72).to(dtype)
    g = torch.Generator().manual_seed(73)
    pm = torch.rand(B, N, N, generator=g) > 0.15
    args = (w.ln_pair_weight, w.ln_pair_bias, torch.cat([w.to_left, w.to_right]),
            torch.cat([w.to_left_gate, w.to_right_gate]), w.ln_out_weight, w.ln_out_bias, w.to_out, w.to_gate)
    ref = O.trimul_forward_functional(z, direction, pm, *args).float()
    y = f(z.to(dev), direction, pm.to(dev), *(a.to(dev) for a in args)).cpu().float()
    assert read_status(dev)[0] == 0
    assert tuple(y.shape) == (B, N, N, d)
    err = O.rel_rms(y, ref)
    assert err <= (TOL_FP32 if dtype == torch.float32 else TOL_BF16), f"rel-RMS {err:.3e}"
    with pytest.raises(ValueError):      # odd leading dimension of the packed projections
        f(z.to(dev), direction, None, args[0].to(dev), args[1].to(dev), args[2][:-1].to(dev), args[3][:-1].to(dev),
          *(a.to(dev) for a in args[4:]))


def test_bidirectional_functional_op_has_the_reference_argument_names(dev):
    from miniworld_engine_b200 import bidirectional_triangle_multiplicative_update_b200 as f
    w = O.make_bidir_weights(128, 128, 81, affine="random").to(torch.bfloat16)
    z = O.make_input(1, 96, 128, 82).bfloat16()
    m = O.make_token_mask(1, 96, "tail9")
    t = lambda x: x.to(dev)
    y = f(t(z), t(m), norm_in_weight=t(w.ln_pair_weight), norm_in_bias=t(w.ln_pair_bias), to_left_weight=t(w.to_left),
          to_left_gate_weight=t(w.to_left_gate), to_right_weight=t(w.to_right),
          to_right_gate_weight=t(w.to_right_gate), norm_out_weight=t(w.ln_out_weight),
          norm_out_bias=t(w.ln_out_bias), to_out_weight=t(w.to_out), to_gate_weight=t(w.to_gate)).cpu().float()
    ref = O.bidir_forward(z, m, w, add_residual=False).float()
    assert O.rel_rms(y, ref) <= TOL_BF16


def test_bidirectional_module_mirrors_the_reference_interface(dev):
    from miniworld_engine_b200 import BidirectionalTriangleMultiplicationB200
    w = O.make_bidir_weights(128, 128, 11)
    mod = BidirectionalTriangleMultiplicationB200(128)
    assert set(mod.state_dict().keys()) == set(w.state_dict().keys())
    # freshly constructed: gates and to_out are zero, so the block returns its input (residual only)
    z = O.make_input(1, 64, 128, 2).bfloat16().to(dev)
    fresh = BidirectionalTriangleMultiplicationB200(128).to(dev).to(torch.bfloat16).eval()
    with torch.no_grad():
        assert torch.equal(fresh(z), z)
    mod.load_state_dict(w.state_dict())
    mod = mod.to(dev).to(torch.bfloat16).eval()
    assert mod.ln_pair.weight.dtype == torch.float32 and mod.ln_out.weight.shape == (256,)
    with torch.no_grad():
        y = mod(z).float().cpu()
    ref = O.bidir_forward(z.cpu(), None, w.to(torch.bfloat16)).float()
    assert O.rel_rms(y, ref) <= TOL_BF16
    with pytest.raises(NotImplementedError):
        mod(z.requires_grad_(True))


def test_bidirectional_entry_point_equals_the_stage_calls_it_is_made_of(dev):
    """trimul_b200_forward_bidir = stage 1 per direction with its rows of the [2h, d] weights, one
    contraction over 2h planes, the wide last stage: assembling the same calls by hand must give
    the same bits."""
    from miniworld_engine_b200 import stages as S
    N, d = 160, 128
    w = O.make_bidir_weights(d, d, 21, affine="random").to(torch.bfloat16)
    z = O.make_input(1, N, d, 22).bfloat16().to(dev)
    m = O.make_token_mask(1, N, "tail11").to(dev)
    y = run_bidir(z.cpu().float(), m.cpu(), w, torch.bfloat16, dev)
    t = lambda x: x.to(dev)
    a = S.alloc_planes(2 * d, N, N, torch.bfloat16, dev)
    b = S.alloc_planes(2 * d, N, N, torch.bfloat16, dev)
    tri = S.alloc_planes(2 * d, N, N, torch.bfloat16, dev)
    w_gate = t(w.to_gate)
    for direction in (0, 1):
        rows = slice(direction * d, (direction + 1) * d)
        first = direction * d * a.plane_stride
        va, vb = (S.PlaneSpec(sp.buf[first:], d, N, N, sp.pitch, sp.plane_stride) for sp in (a, b))
        wd = dict(ln_in_w=t(w.ln_pair_weight), ln_in_b=t(w.ln_pair_bias), w_left=t(w.to_left)[rows],
                  w_left_gate=t(w.to_left_gate)[rows], w_right=t(w.to_right)[rows],
                  w_right_gate=t(w.to_right_gate)[rows], ln_out_w=t(w.ln_pair_weight), ln_out_b=t(w.ln_pair_bias),
                  w_gate=w_gate, w_out=w_gate)
        S.tm1(z, m, wd, va, vb, outgoing=(direction == 0))
    S.contract(a, b, tri)
    wd3 = dict(ln_in_w=t(w.ln_pair_weight), ln_in_b=t(w.ln_pair_bias), w_left=w_gate, w_left_gate=w_gate,
               w_right=w_gate, w_right_gate=w_gate, ln_out_w=t(w.ln_out_weight), ln_out_b=t(w.ln_out_bias),
               w_gate=w_gate, w_out=t(w.to_out))
    y2 = S.tm2(z, tri, wd3, residual=z).cpu()
    assert torch.equal(y, y2)


def test_full_size_symmetric_input_makes_both_directions_identical(dev):
    """Size-independent property, checked at a full benchmark size (N = 1024, no oracle run needed):
    for a pair tensor with z[i,j] = z[j,i] the incoming operands a'[i][k] = a[k,i] equal the outgoing
    ones bit for bit, the contraction sums over k in the same order, and the last stage is the
    same — so the two directions must return identical tensors."""
    N = 1024
    w = O.make_weights(128, 4, affine="random")
    g = torch.Generator().manual_seed(12)
    z = torch.randn(1, N, N, 128, generator=g)
    z = (0.5 * (z + z.transpose(1, 2))).bfloat16()
    assert torch.equal(z, z.transpose(1, 2))
    m = O.make_token_mask(1, N, "rand5", seed=3)
    out = run_block(z.float(), m, w, True, torch.bfloat16, dev)
    inc = run_block(z.float(), m, w, False, torch.bfloat16, dev)
    assert torch.equal(out, inc)
    assert float(out.float().abs().max()) > 0


def test_full_size_token_permutation_equivariance(dev):
    """Relabelling the tokens (z'[i,j] = z[p(i),p(j)], mask' = mask[p]) must relabel the output the
    same way; only the order of the k-summation changes, so the agreement is to accumulation
    noise, far inside the bf16 tolerance.  N = 768, the headline size."""
    N = 768
    w = O.make_weights(128, 0)
    z = O.make_input(1, N, 128, 1).bfloat16()
    m = O.make_token_mask(1, N, "tail77")
    p = torch.randperm(N, generator=torch.Generator().manual_seed(8))
    zp = z[:, p][:, :, p].contiguous()
    for outgoing in (True, False):
        y = run_block(z.float(), m, w, outgoing, torch.bfloat16, dev)
        yp = run_block(zp.float(), m[:, p], w, outgoing, torch.bfloat16, dev)
        err = O.rel_rms(yp.float(), y[:, p][:, :, p].float())
        assert err <= 3e-3, f"outgoing={outgoing}: rel-RMS {err:.3e}"


def test_headline_n768_outgoing_vs_oracle(dev):
    """The benchmark's headline workload itself (bf16, B=1, N=768, c=128, outgoing, all-ones token
    mask) against the CPU oracle on the same seeded inputs."""
    torch.set_num_threads(os.cpu_count() or 1)
    w, z, m = O.make_weights(128, 0), O.make_input(1, 768, 128, 1), O.make_token_mask(1, 768, "ones")
    y = run_block(z, m, w, True, torch.bfloat16, dev)
    ref = oracle_out(z, m, w, True, torch.bfloat16)
    err = O.rel_rms(y.float(), ref.float())
    assert err <= TOL_BF16, f"rel-RMS {err:.3e}"


def test_config5_n2048_outgoing_then_incoming_vs_oracle(dev):
    """BASELINE config 5 on one GPU: an outgoing block followed by an incoming block on its output
    (independent weight sets, seeds 0 and 3), N=2048, random 5 % token padding, against two CPU-oracle
    block calls.  The second block is compared on the SAME input (the first block's GPU output), so the
    check is per block and errors do not compound."""
    torch.set_num_threads(os.cpu_count() or 1)
    N = 2048
    w1, w2 = O.make_weights(128, 0), O.make_weights(128, 3)
    z, m = O.make_input(1, N, 128, 1), O.make_token_mask(1, N, "rand5")
    y1 = run_block(z, m, w1, True, torch.bfloat16, dev)
    ref1 = oracle_out(z, m, w1, True, torch.bfloat16)
    e1 = O.rel_rms(y1.float(), ref1.float())
    assert e1 <= TOL_BF16, f"outgoing block: rel-RMS {e1:.3e}"
    del ref1
    y2 = run_block(y1.float(), m, w2, False, torch.bfloat16, dev)
    ref2 = O.trimul_forward(y1, m, w2.to(torch.bfloat16), False)
    e2 = O.rel_rms(y2.float(), ref2.float())
    assert e2 <= TOL_BF16, f"incoming block: rel-RMS {e2:.3e}"
    # padded output rows of the second block: LayerNorm_out of an all-zero contraction gives beta = 0
    pad = ~m[0]
    assert float(y2[0, pad].abs().max()) == 0.0 and float(y2[0, :, pad].abs().max()) == 0.0


def test_fused_dropout_scale_equals_the_unfused_composition(dev):
    """`block * scale + pair` fused into the last stage's epilogue gives bit for bit what the three
    separate operations give (same rounding points), on the tensor-core path and on the others."""
    from miniworld_engine_b200 import read_status, trimul_forward
    for c, N, dtype in ((128, 200, torch.bfloat16), (64, 40, torch.bfloat16), (32, 24, torch.float32)):
        w = O.make_weights(c, 5, affine="random")
        z = O.make_input(2, N, c, 6).to(dtype).to(dev)
        m = O.make_token_mask(2, N, "tail9").to(dev)
        g = torch.Generator().manual_seed(7)
        ds = ((torch.rand(2, 1, N, c, generator=g) > 0.3).float() / 0.7).to(dtype).to(dev)
        kw = forward_kwargs(w, dtype, dev)
        fused = trimul_forward(z, m, outgoing=True, **kw, residual=z, drop_scale=ds)
        plain = trimul_forward(z, m, outgoing=True, **kw)
        assert torch.equal(fused, plain * ds + z), (c, N, dtype)
        only_scale = trimul_forward(z, m, outgoing=True, **kw, drop_scale=ds)
        assert torch.equal(only_scale, plain * ds), (c, N, dtype)
    assert read_status(dev)[0] == 0


def test_contraction_refuses_a_ragged_last_k_chunk_on_the_tensor_cores(dev):
    """K-chunked operands (what an all-to-all leaves behind) whose last chunk is not full: the
    tensor-core kernel would read the chunk's padding, so the call must take the CUDA-core kernel,
    which bounds every index.  The padding is poisoned with NaN to prove nothing reads it."""
    from miniworld_engine_b200 import stages as S
    P, R, K, chunk = 8, 128, 192, 128
    g = torch.Generator().manual_seed(3)
    a_d = torch.randn(P, R, K, generator=g).bfloat16().to(dev)
    b_d = torch.randn(P, R, K, generator=g).bfloat16().to(dev)
    a = S.alloc_planes(P, R, K, torch.bfloat16, dev, fill=float("nan"), col_chunk=chunk)
    b = S.alloc_planes(P, R, K, torch.bfloat16, dev, fill=float("nan"), col_chunk=chunk)
    # the test helper scatters whole chunks only: fill chunk 0 fully, chunk 1 with the remaining 64 columns
    for spec, dense in ((a, a_d), (b, b_d)):
        v = spec.buf[: 2 * spec.chunk_stride].view(2, P, R, spec.pitch)
        v[0, :, :, :chunk] = dense[..., :chunk]
        v[1, :, :, : K - chunk] = dense[..., chunk:]
    t = S.alloc_planes(P, R, R, torch.bfloat16, dev, fill=float("nan"))
    S.contract(a, b, t)
    got = S.planes_to_dense(t).float()
    ref = torch.einsum("pik,pjk->pij", a_d.float(), b_d.float())
    assert not torch.isnan(got).any()
    assert O.rel_rms(got.cpu(), ref.cpu()) <= 5e-3


def test_serial_launch_gives_the_same_result(dev):
    """Programmatic dependent launch only moves the start of a stage's set-up: with it (default) and
    without it (TRIMUL_FLAG_SERIAL_LAUNCH) the block output is bit-identical, also when calls follow
    each other back to back and reuse the same workspace."""
    from miniworld_engine_b200 import read_status, trimul_forward
    for c, N in ((128, 200), (256, 72), (64, 136)):
        w = O.make_weights(c, 0, affine="random")
        z = O.make_input(1, N, c, 1).bfloat16().to(dev)
        m = O.make_token_mask(1, N, "tail9").to(dev)
        kw = forward_kwargs(w, torch.bfloat16, dev)
        outs = [trimul_forward(z, m, outgoing=(i % 2 == 0), **kw, residual=z) for i in range(6)]
        for i, y in enumerate(outs):
            y_serial = trimul_forward(z, m, outgoing=(i % 2 == 0), **kw, residual=z, serial_launch=True)
            assert torch.equal(y, y_serial), (c, N, i)
    assert read_status(dev)[0] == 0


def test_randomised_shapes_kernel_variants_agree_bit_for_bit(dev):
    """Random batch sizes, token counts (multiples of nothing in particular), mask kinds and directions:
    the CTA-pair and lone-CTA forms of stage 1 and of the contraction give identical bits, repeated calls
    reproduce themselves, nothing but the planes is written (NaN-filled scratch), every value is finite
    and no bounded wait expires."""
    import random
    from miniworld_engine_b200 import read_status, stages as S
    from tests._util import weights_dict
    rng = random.Random(7)
    gen = torch.Generator().manual_seed(7)
    w = O.make_weights(128, 0, affine="random")
    wd = weights_dict(w, torch.bfloat16, dev)
    for _ in range(16):
        B, N = rng.choice([1, 1, 2, 3]), rng.choice([16, 33, 64, 100, 128, 191, 256, 300, 384])
        z = torch.randn(B, N, N, 128, generator=gen).bfloat16().to(dev)
        kind = rng.choice(["none", "token", "pair"])
        m = None if kind == "none" else (torch.rand((B, N) if kind == "token" else (B, N, N), generator=gen) > 0.2).to(dev)
        outgoing = rng.choice([True, False])
        res = []
        for single_cta in (False, True, False):
            a = S.alloc_planes(B * 128, N, N, torch.bfloat16, dev, fill=float("nan"))
            b = S.alloc_planes(B * 128, N, N, torch.bfloat16, dev, fill=float("nan"))
            S.tm1(z, m, wd, a, b, outgoing=outgoing, single_cta=single_cta)
            res.append((S.planes_to_dense(a).clone(), S.planes_to_dense(b).clone(), a, b))
        for k in (1, 2):
            assert torch.equal(res[0][0], res[k][0]) and torch.equal(res[0][1], res[k][1]), (B, N, kind, outgoing, k)
        assert bool(torch.isfinite(res[0][0].float()).all()) and bool(torch.isfinite(res[0][1].float()).all())
        t1 = S.alloc_planes(B * 128, N, N, torch.bfloat16, dev, fill=float("nan"))
        t2 = S.alloc_planes(B * 128, N, N, torch.bfloat16, dev, fill=float("nan"))
        S.contract(res[0][2], res[0][3], t1)
        S.contract(res[0][2], res[0][3], t2, single_cta=True)
        assert torch.equal(S.planes_to_dense(t1), S.planes_to_dense(t2)), (B, N, kind, outgoing)
        y = S.tm2(z, t1, wd)
        assert torch.equal(y, S.tm2(z, t1, wd))
        if N <= 128:      # the oracle is quick at these sizes: the stage calls above ARE the block
            w16 = w.to(torch.bfloat16)
            ref = O.trimul_stages(z.cpu(), None if kind != "token" else m.cpu(), w16, outgoing,
                                  pair_mask=m.cpu() if kind == "pair" else None)["out"]
            assert O.rel_rms(y.float().cpu(), ref.float()) <= TOL_BF16, (B, N, kind, outgoing)
    assert read_status(dev)[0] == 0
