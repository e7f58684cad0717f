"""Row-sharded block on the GPU.

* One-GPU emulation: every rank's stage 1, contraction and stage 3 run one after the other on
  ``cuda:0`` and the exchange is done with plain copies into the same chunk-major buffers the
  collectives fill.  This exercises the kernels' chunked operand addressing (row-chunked and
  k-chunked tensor maps) without needing several GPUs.
* Real multi-GPU run (NCCL, one process per GPU) when at least two devices are visible.

Tolerance: rel-RMS <= 1e-2 against the bf16 oracle; the slabs must also agree with the unsharded
GPU result to within the tensor-core / CUDA-core kernel difference (4e-3), and bit for bit when
both took the same kernels.
"""

import os
import socket
import subprocess
import sys

import pytest
import torch

from oracle import trimul_oracle as O
from tests._util import forward_kwargs, weights_dict

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _emulated_sharded(z, m, w, outgoing, world, dev):
    from miniworld_engine_b200 import stages as S
    from miniworld_engine_b200.sharded import ShardPlan
    B, N, _, c = z.shape
    wd = weights_dict(w, torch.bfloat16, dev)
    zd, md = z.bfloat16().to(dev), m.to(dev)
    plans = [ShardPlan(B, N, c, world, r, outgoing) for r in range(world)]
    bufs = [p.alloc(torch.bfloat16, dev) for p in plans]
    b_shared = bufs[0][2]
    for t in (b_shared, *[bf[0] for bf in bufs], *[bf[1] for bf in bufs]):
        t.view(torch.int16).fill_(0x7FC0)                       # NaN: unwritten data must not be read
    R = plans[0].R
    for r, p in enumerate(plans):                                # stage 1 of every rank
        a_w, b_w = p.tm1_outputs(bufs[r][0], b_shared)
        S.tm1(zd[:, r * R:(r + 1) * R].contiguous(), md, wd, a_w, b_w, outgoing=outgoing, row0=p.row0)
    if not outgoing:                                             # the all-to-all, by hand
        n = plans[0].a2a_chunk_elems()
        for r in range(world):
            for s in range(world):
                bufs[r][1][s * n:(s + 1) * n].copy_(bufs[s][0][r * n:(r + 1) * n])
    outs = []
    for r, p in enumerate(plans):
        a_r, b_r = p.contract_operands(bufs[r][1], b_shared)
        tri = p.tri_spec(bufs[r][3])
        S.contract(a_r, b_r, tri)
        outs.append(S.tm2(zd[:, r * R:(r + 1) * R].contiguous(), tri, wd, row0=p.row0))
    return torch.cat(outs, dim=1).cpu()


def _emulated_channel_sharded(z, m, w, outgoing, world, dev):
    """Same, for the channel-sharded contraction: three all-to-alls done as chunk copies."""
    from miniworld_engine_b200 import stages as S
    from miniworld_engine_b200.sharded import ChannelShardPlan
    B, N, _, c = z.shape
    wd = weights_dict(w, torch.bfloat16, dev)
    zd, md = z.bfloat16().to(dev), m.to(dev)
    plans = [ChannelShardPlan(B, N, c, world, r, outgoing) for r in range(world)]
    bufs = [p.alloc(torch.bfloat16, dev) for p in plans]
    for bf in bufs:
        for t in bf.values():
            t.view(torch.int16).fill_(0x7FC0)
    R = plans[0].R
    for r, p in enumerate(plans):
        a_w, b_w = p.tm1_outputs(bufs[r])
        S.tm1(zd[:, r * R:(r + 1) * R].contiguous(), md, wd, a_w, b_w, outgoing=outgoing, row0=p.row0)

    def all_to_all(src, dst):
        n = bufs[0][src].numel() // world
        for r in range(world):
            for s in range(world):
                bufs[r][dst][s * n:(s + 1) * n].copy_(bufs[s][src][r * n:(r + 1) * n])

    all_to_all("a_send", "a_recv")
    all_to_all("b_send", "b_recv")
    for r, p in enumerate(plans):
        a_r, b_r, tri_w = p.contract_operands(bufs[r])
        S.contract(a_r, b_r, tri_w)
    all_to_all("tri_send", "tri_recv")
    outs = [S.tm2(zd[:, r * R:(r + 1) * R].contiguous(), p.tri_spec(bufs[r]), wd, row0=p.row0)
            for r, p in enumerate(plans)]
    return torch.cat(outs, dim=1).cpu()


def _emulated_peer_sharded(z, m, w, outgoing, world, dev):
    """The collective-free variant: every virtual rank's scattering stage 1 and scattering
    contraction store straight into the receive buffers of all virtual ranks (here: buffers on the
    same GPU; on several GPUs the same pointers are peer mappings)."""
    from miniworld_engine_b200 import stages as S
    from miniworld_engine_b200.sharded import ChannelShardPlan, peer_dest_specs
    B, N, _, c = z.shape
    wd = weights_dict(w, torch.bfloat16, dev)
    zd, md = z.bfloat16().to(dev), m.to(dev)
    plans = [ChannelShardPlan(B, N, c, world, r, outgoing) for r in range(world)]
    bufs = [p.alloc(torch.bfloat16, dev) for p in plans]
    for bf in bufs:
        for t in bf.values():
            t.view(torch.int16).fill_(0x7FC0)
    R = plans[0].R
    dests = [peer_dest_specs(p, lambda d: bufs[d]["a_recv"], lambda d: bufs[d]["b_recv"],
                             lambda d: bufs[d]["tri_recv"]) for p in plans]
    for r, p in enumerate(plans):
        S.tm1_scatter(zd[:, r * R:(r + 1) * R].contiguous(), md, wd, dests[r][0], dests[r][1],
                      outgoing=outgoing, row0=p.row0)
    for r, p in enumerate(plans):
        a_r, b_r, _ = p.contract_operands(bufs[r])
        S.contract_scatter(a_r, b_r, dests[r][2])
    outs = [S.tm2(zd[:, r * R:(r + 1) * R].contiguous(), p.tri_spec(bufs[r]), wd, row0=p.row0)
            for r, p in enumerate(plans)]
    return torch.cat(outs, dim=1).cpu()


@pytest.mark.parametrize("B,N,world", [(1, 512, 2), (1, 512, 4), (2, 256, 2)])
@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
def test_one_gpu_emulation_of_peer_scatter(outgoing, B, N, world):
    from miniworld_engine_b200 import read_status, trimul_forward
    dev = torch.device("cuda", 0)
    w = O.make_weights(128, 0, affine="random")
    z = O.make_input(B, N, 128, 1)
    m = O.make_token_mask(B, N, "rand5")
    got = _emulated_peer_sharded(z, m, w, outgoing, world, dev)
    assert read_status(dev)[0] == 0
    whole = trimul_forward(z.bfloat16().to(dev), m.to(dev), outgoing=outgoing,
                           **forward_kwargs(w, torch.bfloat16, dev)).cpu()
    assert not torch.isnan(got.float()).any()
    assert torch.equal(got, whole)          # same kernels, same accumulation order


def test_scatter_entry_points_reject_what_they_cannot_do():
    from miniworld_engine_b200 import stages as S
    from miniworld_engine_b200.sharded import ChannelShardPlan, peer_dest_specs
    dev = torch.device("cuda", 0)
    w = O.make_weights(128, 0)
    # fp32 has no scattering kernel
    wd32 = weights_dict(w, torch.float32, dev)
    p = ChannelShardPlan(1, 256, 128, 2, 0, True)
    bufs = p.alloc(torch.float32, dev)
    d = peer_dest_specs(p, lambda k: bufs["a_recv"], lambda k: bufs["b_recv"], lambda k: bufs["tri_recv"])
    z = torch.zeros(1, 128, 256, 128, device=dev)
    with pytest.raises(NotImplementedError):
        S.tm1_scatter(z, None, wd32, d[0], d[1], outgoing=True)
    # R = 64 rows per destination: a contraction tile would straddle two destinations
    wd = weights_dict(w, torch.bfloat16, dev)
    p = ChannelShardPlan(1, 256, 128, 4, 0, True)
    bufs = p.alloc(torch.bfloat16, dev)
    d = peer_dest_specs(p, lambda k: bufs["a_recv"], lambda k: bufs["b_recv"], lambda k: bufs["tri_recv"])
    a_r, b_r, _ = p.contract_operands(bufs)
    with pytest.raises(NotImplementedError):
        S.contract_scatter(a_r, b_r, d[2])


@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
def test_one_gpu_emulation_of_channel_sharding(outgoing):
    from miniworld_engine_b200 import read_status, trimul_forward
    dev = torch.device("cuda", 0)
    N, world = 512, 2
    w = O.make_weights(128, 0, affine="random")
    z = O.make_input(1, N, 128, 1)
    m = O.make_token_mask(1, N, "rand5")
    got = _emulated_channel_sharded(z, m, w, outgoing, world, dev)
    assert read_status(dev)[0] == 0
    whole = trimul_forward(z.bfloat16().to(dev), m.to(dev), outgoing=outgoing,
                           **forward_kwargs(w, torch.bfloat16, dev)).cpu()
    assert not torch.isnan(got.float()).any()
    assert torch.equal(got, whole)          # same kernels, same accumulation order


@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
@pytest.mark.parametrize("N,world", [(512, 2), (256, 4)])
def test_one_gpu_emulation_of_row_sharding(N, world, outgoing):
    from miniworld_engine_b200 import read_status, trimul_forward
    dev = torch.device("cuda", 0)
    w = O.make_weights(128, 0, affine="random")
    z = O.make_input(1, N, 128, 1)
    m = O.make_token_mask(1, N, "rand5")
    got = _emulated_sharded(z, m, w, outgoing, world, dev)
    assert read_status(dev)[0] == 0
    whole = trimul_forward(z.bfloat16().to(dev), m.to(dev), outgoing=outgoing,
                           **forward_kwargs(w, torch.bfloat16, dev)).cpu()
    ref = O.trimul_forward(z.bfloat16(), m, w.to(torch.bfloat16), outgoing)
    assert not torch.isnan(got.float()).any()
    assert O.rel_rms(got.float(), whole.float()) <= 4e-3
    assert O.rel_rms(got.float(), ref.float()) <= 1e-2
    if N == 512:   # every stage took the tensor-core kernels in both runs: identical arithmetic
        assert torch.equal(got, whole)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("mode", ["rows", "channels", "peer"])
@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
def test_nccl_row_sharding_matches_single_gpu(outgoing, mode):
    world = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "sharded_worker.py"), "--N", "512", "--direction",
           "outgoing" if outgoing else "incoming", "--mode", mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=220, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "SHARDED_OK" in res.stdout
