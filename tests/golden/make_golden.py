"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference tree is available (it cannot travel to a GPU box):

    python tests/golden/make_golden.py --reference /path/to/miniworld-engine

It imports the reference's ``TriangleMultiplicationReference``,
``triangle_multiplicative_update_pytorch``
(``src/miniworld_engine/modules/triangle_multiplication/reference.py:32-122``) and
``BidirectionalTriangleMultiplication`` (``.../bidirectional.py:93-156``, eager branch) and the
``TriangleMultiplication`` module in training mode with row-broadcast dropout
(``.../module.py:208-222,332-337``, PyTorch backend) unmodified,
runs them on CPU on the seeded inputs produced by ``oracle/trimul_oracle.py``'s
generators, and writes one ``.npz`` per case: the inputs actually fed (so a
change in a random generator cannot silently move the fixture) and the
reference's output.  bf16 results are stored widened to fp32 (exact).
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import trimul_oracle as O  # noqa: E402

# name, form, dtype, B, N, c, direction, mask kind, affine, weight seed, input seed
CASES = [
    ("cfg1_out_fp32_n32_c128", "module", "fp32", 1, 32, 128, "outgoing", "ones", "unit", 0, 1),
    ("out_fp32_n12_c32_tail3_aff", "module", "fp32", 2, 12, 32, "outgoing", "tail3", "random", 10, 11),
    ("in_fp32_n12_c32_tail3_aff", "module", "fp32", 2, 12, 32, "incoming", "tail3", "random", 10, 11),
    ("in_fp32_n13_c64_nomask", "module", "fp32", 1, 13, 64, "incoming", "none", "random", 12, 13),
    ("out_bf16_n16_c64_tail5_aff", "module", "bf16", 1, 16, 64, "outgoing", "tail5", "random", 20, 21),
    ("in_bf16_n16_c64_rand5", "module", "bf16", 2, 16, 64, "incoming", "rand5", "unit", 22, 23),
    ("out_bf16_n24_c128_ones", "module", "bf16", 1, 24, 128, "outgoing", "ones", "unit", 0, 1),
    ("func_out_fp32_n10_c32_pairmask", "functional", "fp32", 2, 10, 32, "outgoing", "pair", "random", 30, 31),
    ("func_in_bf16_n10_c32_pairmask", "functional", "bf16", 1, 10, 32, "incoming", "pair", "random", 32, 33),
]


# bidirectional module (bidirectional.py:93-156): name, dtype, B, N, d, mask kind, affine, weight seed,
# input seed[, d_hidden (default d)]
BIDIR_CASES = [
    ("bidir_fp32_n12_d32_tail3_aff", "fp32", 2, 12, 32, "tail3", "random", 40, 41),
    ("bidir_bf16_n16_d64_rand5_aff", "bf16", 1, 16, 64, "rand5", "random", 42, 43),
    ("bidir_bf16_n20_d128_nomask", "bf16", 1, 20, 128, "none", "unit", 44, 45),
    ("bidir_fp32_n11_d32_h16_tail3_aff", "fp32", 2, 11, 32, "tail3", "random", 46, 47, 16),
    ("bidir_bf16_n14_d128_h64_rand5_aff", "bf16", 1, 14, 128, "rand5", "random", 48, 49, 64),
    ("bidir_bf16_n12_d64_h128_tail2_aff", "bf16", 1, 12, 64, "tail2", "random", 50, 51, 128),
]


# the MODULE in training mode with row-broadcast dropout (module.py:208-222,332-337), generic PyTorch
# backend: name, dtype, B, N, c, direction, mask kind, affine, weight seed, input seed, p_drop, rng seed
DROPOUT_CASES = [
    ("drop_out_fp32_n12_c32_tail3_aff_p25", "fp32", 2, 12, 32, "outgoing", "tail3", "random", 60, 61, 0.25, 7),
    ("drop_in_bf16_n16_c128_rand5_aff_p15", "bf16", 1, 16, 128, "incoming", "rand5", "random", 62, 63, 0.15, 8),
    ("drop_out_bf16_n14_c64_nomask_p50", "bf16", 2, 14, 64, "outgoing", "none", "unit", 64, 65, 0.5, 9),
]


def run_dropout_reference(case):
    from miniworld_engine.modules.triangle_multiplication.module import TriangleMultiplication
    name, dt, B, N, c, direction, mkind, affine, wseed, zseed, p_drop, rseed = case
    dtype = torch.float32 if dt == "fp32" else torch.bfloat16
    w = O.make_weights(c, wseed, affine=affine)
    z = O.make_input(B, N, c, zseed)
    mask = None if mkind == "none" else O.make_token_mask(B, N, mkind, seed=zseed + 100)
    with torch.no_grad():
        m = TriangleMultiplication(c, outgoing=(direction == "outgoing"), implementation="pytorch", p_drop=p_drop)
        m.load_state_dict(w.state_dict())
        m = m.to(dtype).train()
        zd = z.to(dtype)
        torch.manual_seed(rseed)
        y = m(zd, mask)
        # the scale is the first (and only) draw of the forward pass: the same seed reproduces it
        torch.manual_seed(rseed)
        ds = m._make_drop_row_scale(zd, p_drop)
    return z, mask, w, ds, y


def run_bidir_reference(case):
    from miniworld_engine.modules.triangle_multiplication.bidirectional import BidirectionalTriangleMultiplication
    name, dt, B, N, d, mkind, affine, wseed, zseed = case[:9]
    h = case[9] if len(case) > 9 else d
    dtype = torch.float32 if dt == "fp32" else torch.bfloat16
    w = O.make_bidir_weights(d, h, wseed, affine=affine)
    z = O.make_input(B, N, d, zseed)
    mask = None if mkind == "none" else O.make_token_mask(B, N, mkind, seed=zseed + 100)
    with torch.no_grad():
        m = BidirectionalTriangleMultiplication(d, h)
        m.load_state_dict(w.state_dict())
        m = m.to(dtype).eval()
        y = m(z.to(dtype), mask)
    return z, mask, w, y


def build_case(case):
    name, form, dt, B, N, c, direction, mkind, affine, wseed, zseed = case
    dtype = torch.float32 if dt == "fp32" else torch.bfloat16
    w = O.make_weights(c, wseed, affine=affine)
    z = O.make_input(B, N, c, zseed)
    if mkind == "none":
        mask = None
    elif mkind == "pair":
        g = torch.Generator().manual_seed(zseed + 100)
        mask = torch.rand(B, N, N, generator=g) > 0.2
    else:
        mask = O.make_token_mask(B, N, mkind, seed=zseed + 100)
    return dtype, w, z, mask


def run_reference(case, ref_mod):
    name, form, dt, B, N, c, direction, mkind, affine, wseed, zseed = case
    dtype, w, z, mask = build_case(case)
    with torch.no_grad():
        if form == "module":
            m = ref_mod.TriangleMultiplicationReference(c, outgoing=(direction == "outgoing"))
            m.load_state_dict(w.state_dict())
            m = m.to(dtype)
            y = m(z.to(dtype), mask)
        else:
            wd = w.to(dtype)
            y = ref_mod.triangle_multiplicative_update_pytorch(
                z.to(dtype), direction, mask,
                wd.ln_pair_weight, wd.ln_pair_bias,
                torch.cat([wd.to_left, wd.to_right]), torch.cat([wd.to_left_gate, wd.to_right_gate]),
                wd.ln_out_weight, wd.ln_out_bias, wd.to_out, wd.to_gate, 1e-5)
    return z, mask, w, y


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import miniworld_engine.modules.triangle_multiplication.reference as ref_mod

    torch.set_num_threads(1)  # one summation order, whatever machine regenerates these
    for case in CASES:
        name = case[0]
        z, mask, w, y = run_reference(case, ref_mod)
        arrays = {"z": z.numpy(), "out": y.float().numpy()}
        if mask is not None:
            arrays["mask"] = mask.numpy()
        for k, v in w.state_dict().items():
            arrays["w:" + k] = v.numpy()
        if name.startswith("cfg1"):
            # inputs are regenerated from the seeds; keep only a fingerprint of them
            arrays = {"out": arrays["out"],
                      "z_sum": np.float64(z.double().sum().item()),
                      "z_abs_sum": np.float64(z.double().abs().sum().item()),
                      "w_sum": np.float64(sum(v.double().sum().item() for v in w.state_dict().values()))}
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: out shape {tuple(y.shape)} dtype {y.dtype} -> {os.path.getsize(path)} B")
    for case in DROPOUT_CASES:
        name = case[0]
        z, mask, w, ds, y = run_dropout_reference(case)
        arrays = {"z": z.numpy(), "out": y.float().numpy(), "drop_scale": ds.float().numpy()}
        if mask is not None:
            arrays["mask"] = mask.numpy()
        for k, v in w.state_dict().items():
            arrays["w:" + k] = v.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: out shape {tuple(y.shape)} dtype {y.dtype}, kept {float((ds != 0).float().mean()):.2f} -> "
              f"{os.path.getsize(path)} B")
    for case in BIDIR_CASES:
        name = case[0]
        z, mask, w, y = run_bidir_reference(case)
        arrays = {"z": z.numpy(), "out": y.float().numpy()}
        if mask is not None:
            arrays["mask"] = mask.numpy()
        for k, v in w.state_dict().items():
            arrays["w:" + k] = v.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: out shape {tuple(y.shape)} dtype {y.dtype} -> {os.path.getsize(path)} B")


if __name__ == "__main__":
    main()
