"""Helpers shared by the GPU parity tests."""

from __future__ import annotations

import torch

from oracle import trimul_oracle as O


def weights_dict(w: O.TrimulWeights, dtype: torch.dtype, device) -> dict:
    """Oracle parameter set -> keyword dict of device tensors for the stage wrappers.
    ``w`` is cast with the reference's module-cast semantics first."""
    wd = w.to(dtype)
    return dict(
        ln_in_w=wd.ln_pair_weight.to(device), ln_in_b=wd.ln_pair_bias.to(device),
        w_left=wd.to_left.to(device), w_left_gate=wd.to_left_gate.to(device),
        w_right=wd.to_right.to(device), w_right_gate=wd.to_right_gate.to(device),
        ln_out_w=wd.ln_out_weight.to(device), ln_out_b=wd.ln_out_bias.to(device),
        w_gate=wd.to_gate.to(device), w_out=wd.to_out.to(device))


def forward_kwargs(w: O.TrimulWeights, dtype: torch.dtype, device) -> dict:
    d = weights_dict(w, dtype, device)
    return dict(
        ln_in_weight=d["ln_in_w"], ln_in_bias=d["ln_in_b"], w_left=d["w_left"], w_left_gate=d["w_left_gate"],
        w_right=d["w_right"], w_right_gate=d["w_right_gate"], ln_out_weight=d["ln_out_w"],
        ln_out_bias=d["ln_out_b"], w_gate=d["w_gate"], w_out=d["w_out"],
        eps_in=w.eps_in, eps_out=w.eps_out)


def oracle_out(z, mask, w, outgoing, dtype):
    """Oracle output for activations of ``dtype`` (inputs given in fp32)."""
    return O.trimul_forward(z.to(dtype), mask, w.to(dtype), outgoing)
