"""The CPU oracle restates the reference exactly: check it against the golden
fixtures that ``tests/golden/make_golden.py`` produced by running the reference's
own ``reference.py`` (module and functional forms), its bidirectional module and its
``TriangleMultiplication`` module in training mode with row-broadcast dropout."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle import trimul_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
FILES = sorted(glob.glob(os.path.join(GOLD, "*.npz")))


def _weights(d, prefix="w:"):
    g = lambda k: torch.from_numpy(d[prefix + k])
    return O.TrimulWeights(
        g("ln_pair.weight"), g("ln_pair.bias"), g("to_left.weight"), g("to_left_gate.weight"),
        g("to_right.weight"), g("to_right_gate.weight"), g("ln_out.weight"), g("ln_out.bias"),
        g("to_gate.weight"), g("to_out.weight"))


def load_case(path):
    """Returns (name, z fp32, mask or None, weights fp32, golden out fp32, dtype, direction, form)."""
    name = os.path.basename(path)[:-4]
    d = np.load(path)
    if name.startswith("cfg1"):
        w = O.make_weights(128, 0)
        z = O.make_input(1, 32, 128, 1)
        # the generators must still produce what the fixture was made from
        assert abs(z.double().sum().item() - float(d["z_sum"])) < 1e-6
        assert abs(z.double().abs().sum().item() - float(d["z_abs_sum"])) < 1e-6
        assert abs(sum(v.double().sum().item() for v in w.state_dict().values()) - float(d["w_sum"])) < 1e-6
        mask = O.make_token_mask(1, 32, "ones")
    else:
        w = _weights(d)
        z = torch.from_numpy(d["z"])
        mask = torch.from_numpy(d["mask"]) if "mask" in d.files else None
    dtype = torch.bfloat16 if "bf16" in name else torch.float32
    direction = "incoming" if ("in_" in name.split("fp32")[0].split("bf16")[0]) else "outgoing"
    form = ("functional" if name.startswith("func") else "bidir" if name.startswith("bidir") else
            "dropout" if name.startswith("drop") else "module")
    if form == "dropout":
        direction = "incoming" if name.startswith("drop_in") else "outgoing"
    return name, z, mask, w, torch.from_numpy(d["out"]), dtype, direction, form


def load_drop_scale(path, dtype):
    """The row-broadcast dropout scale [B, 1, N, c] the reference module drew for a dropout fixture."""
    return torch.from_numpy(np.load(path)["drop_scale"]).to(dtype)


def test_fixture_set_is_complete():
    names = {os.path.basename(f)[:-4] for f in FILES}
    assert "cfg1_out_fp32_n32_c128" in names
    assert len(names) >= 15
    assert sum(n.startswith("bidir") for n in names) >= 6
    assert sum("_h" in n for n in names) >= 3      # d_hidden != d_pair
    assert sum(n.startswith("drop") for n in names) >= 3   # module in training mode, dropout scale live


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f)[:-4] for f in FILES])
def test_oracle_matches_reference_output(path):
    torch.set_num_threads(1)
    name, z, mask, w, gold, dtype, direction, form = load_case(path)
    wd = w.to(dtype)
    if form == "module":
        y = O.trimul_forward(z.to(dtype), mask, wd, outgoing=(direction == "outgoing"))
    elif form == "bidir":
        y = O.bidir_forward(z.to(dtype), mask, wd)
    elif form == "dropout":
        ds = load_drop_scale(path, dtype)
        assert tuple(ds.shape) == (z.shape[0], 1, z.shape[2], z.shape[3]) and 0.0 < float((ds == 0).float().mean()) < 1.0
        y = O.trimul_module_forward(z.to(dtype), mask, wd, outgoing=(direction == "outgoing"), drop_scale=ds)
    else:
        y = O.trimul_forward_functional(
            z.to(dtype), direction, mask, wd.ln_pair_weight, wd.ln_pair_bias,
            torch.cat([wd.to_left, wd.to_right]), torch.cat([wd.to_left_gate, wd.to_right_gate]),
            wd.ln_out_weight, wd.ln_out_bias, wd.to_out, wd.to_gate, 1e-5)
    assert y.dtype == dtype and tuple(y.shape) == tuple(gold.shape)
    err = O.rel_rms(y.float(), gold)
    # same ops in the same order on the same machine class: equal up to BLAS blocking
    tol = 2e-6 if dtype == torch.float32 else 2e-3
    assert err <= tol, f"{name}: rel-RMS {err:.3e}"
    assert float(gold.abs().max()) > 0  # fixtures are not trivially zero


def test_functional_rejects_bad_direction():
    w = O.make_weights(8, 0)
    z = O.make_input(1, 4, 8, 1)
    with pytest.raises(ValueError):
        O.trimul_forward_functional(
            z, "sideways", None, w.ln_pair_weight, w.ln_pair_bias,
            torch.cat([w.to_left, w.to_right]), torch.cat([w.to_left_gate, w.to_right_gate]),
            w.ln_out_weight, w.ln_out_bias, w.to_out, w.to_gate)


def test_token_mask_equals_outer_product_pair_mask():
    w = O.make_weights(16, 3, affine="random")
    z = O.make_input(1, 9, 16, 4)
    m = O.make_token_mask(1, 9, "tail2")
    pm = m.unsqueeze(-1) & m.unsqueeze(-2)
    for outgoing in (True, False):
        a = O.trimul_stages(z, m, w, outgoing)["out"]
        b = O.trimul_stages(z, None, w, outgoing, pair_mask=pm)["out"]
        assert torch.equal(a, b)
