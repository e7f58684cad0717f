"""Host logic of the row-sharded block on CPU: the exchange step runs over real
``torch.distributed`` collectives (gloo, world size 2 and 4, one process per rank), stage 1 and
stage 2 are played by the CPU oracle writing/reading the very operand-plane layouts the GPU
kernels use.  Every rank must end up with exactly the rows of the contraction it owns."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miniworld_engine_b200 import stages as S
from miniworld_engine_b200.sharded import ChannelShardPlan, ShardPlan, exchange
from oracle import trimul_oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, N, c, B, outgoing, q, mode="rows"):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.set_num_threads(1)
        w = O.make_weights(c, 0, affine="random")
        z = O.make_input(B, N, c, 1)
        m = O.make_token_mask(B, N, "tail3")
        full = O.trimul_stages(z, m, w, outgoing)          # every rank recomputes the truth
        plan = ShardPlan(B, N, c, world, rank, outgoing)
        R, r0 = plan.R, plan.row0
        # stage 1 on the local rows only.  left/right[b, r, s, ch] for z rows r in I_rank.
        left, right = full["left"][:, r0:r0 + R], full["right"][:, r0:r0 + R]
        if outgoing:   # plane element (r, k) = position (r0 + r, k)
            a_d = left.permute(0, 3, 1, 2).reshape(plan.planes, R, N)
            b_d = right.permute(0, 3, 1, 2).reshape(plan.planes, R, N)
        else:          # transposed: plane element (i, k) = position (r0 + k, i)
            a_d = left.permute(0, 3, 2, 1).reshape(plan.planes, N, R)
            b_d = right.permute(0, 3, 2, 1).reshape(plan.planes, N, R)
        want = full["tri"][:, r0:r0 + R].permute(0, 3, 1, 2).reshape(plan.planes, R, N)
        if mode == "channels":
            cp = ChannelShardPlan(B, N, c, world, rank, outgoing)
            bufs = cp.alloc(torch.float32, "cpu")
            for t in bufs.values():
                t.fill_(float("nan"))
            a_w, b_w = cp.tm1_outputs(bufs)
            S.dense_to_planes(a_w, a_d.contiguous())
            S.dense_to_planes(b_w, b_d.contiguous())
            cp.exchange_in(bufs)
            a_r, b_r, tri_w = cp.contract_operands(bufs)
            A, Bm = S.planes_to_dense(a_r), S.planes_to_dense(b_r)
            assert not torch.isnan(A).any() and not torch.isnan(Bm).any()
            S.dense_to_planes(tri_w, torch.einsum("pik,pjk->pij", A, Bm))    # my planes, all rows
            cp.exchange_out(bufs)
            tri = S.planes_to_dense(cp.tri_spec(bufs))                         # all planes, my rows
            err = O.rel_rms(tri, want)
            dist.barrier()
            dist.destroy_process_group()
            q.put((rank, err, None))
            return
        a_send, a_recv, b_full, _ = plan.alloc(torch.float32, "cpu")
        for t in (a_send, a_recv, b_full):
            t.fill_(float("nan"))                          # nothing may be read that was not written
        a_w, b_w = plan.tm1_outputs(a_send, b_full)
        S.dense_to_planes(a_w, a_d.contiguous())
        S.dense_to_planes(b_w, b_d.contiguous())
        exchange(plan, a_send, a_recv, b_full)
        a_r, b_r = plan.contract_operands(a_recv, b_full)
        A, Bm = S.planes_to_dense(a_r), S.planes_to_dense(b_r)
        assert not torch.isnan(A).any() and not torch.isnan(Bm).any()
        tri = torch.einsum("pik,pjk->pij", A, Bm)          # [P][R][N]: rows I_rank of the contraction
        err = O.rel_rms(tri, want)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, err, None))
    except Exception as e:  # pragma: no cover
        q.put((rank, None, repr(e)))


@pytest.mark.parametrize("mode", ["rows", "channels"])
@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
def test_exchange_gives_each_rank_its_rows(world, outgoing, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, 16, 8, 2, outgoing, q, mode))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err, exc in results:
        assert exc is None, f"rank {rank}: {exc}"
        assert err < 1e-6, f"rank {rank}: rel-RMS {err}"


def test_plan_rejects_bad_partitions():
    with pytest.raises(ValueError):
        ShardPlan(1, 10, 8, 4, 0, True)
    with pytest.raises(ValueError):
        ShardPlan(1, 8, 8, 2, 2, True)


def test_channel_plan_rejects_bad_partitions():
    with pytest.raises(ValueError):
        ChannelShardPlan(1, 16, 6, 4, 0, True)      # planes not divisible


def test_single_rank_plan_is_the_plain_layout():
    plan = ShardPlan(1, 24, 8, 1, 0, False)
    a_send, a_recv, b_full, tri = plan.alloc(torch.float32, "cpu")
    assert a_recv is a_send
    a_w, b_w = plan.tm1_outputs(a_send, b_full)
    a_r, b_r = plan.contract_operands(a_recv, b_full)
    for spec in (a_w, b_w, a_r, b_r):
        assert spec.row_chunk is None and spec.col_chunk is None and spec.chunk_stride == 0
    assert (a_r.rows, a_r.cols, b_r.rows, b_r.cols) == (24, 24, 24, 24)


@pytest.mark.parametrize("outgoing", [True, False], ids=["outgoing", "incoming"])
@pytest.mark.parametrize("world", [2, 4])
def test_peer_destinations_are_the_chunks_the_contraction_reads(world, outgoing):
    """The collective-free plan: what rank r's scattering stage 1 writes through its destination
    specs must be exactly what every rank's contraction operands (and stage 3) then read.  The
    scatter itself is emulated with tensor copies: planes [d*P, (d+1)*P) of rank r's stage-1 result
    go to destination d, output rows [d*R, (d+1)*R) of the contraction go to destination d."""
    from miniworld_engine_b200 import stages as S
    from miniworld_engine_b200.sharded import ChannelShardPlan, peer_dest_specs
    B, N, c = 1, 16 * world, 8 * world
    plans = [ChannelShardPlan(B, N, c, world, r, outgoing) for r in range(world)]
    bufs = [p.alloc(torch.float32, "cpu") for p in plans]
    for bf in bufs:
        for t in bf.values():
            t.fill_(float("nan"))
    R, Pp = plans[0].R, plans[0].my_planes
    g = torch.Generator().manual_seed(5)
    # the full operands a[p][i][k] (outgoing) or a'[p][i][k] = a[p][k][i] (incoming), as one array
    a_full = torch.randn(B * c, N, N, generator=g)
    b_full = torch.randn(B * c, N, N, generator=g)
    for r, p in enumerate(plans):
        a_d, b_d, _ = peer_dest_specs(p, lambda d: bufs[d]["a_recv"], lambda d: bufs[d]["b_recv"],
                                      lambda d: bufs[d]["tri_recv"])
        for full, dests in ((a_full, a_d), (b_full, b_d)):
            # stage 1 of rank r produces rows [r*R, (r+1)*R) (outgoing) or k-columns (incoming) of every plane
            mine = full[:, r * R:(r + 1) * R, :] if outgoing else full[:, :, r * R:(r + 1) * R]
            for d in range(world):
                S.dense_to_planes(dests[d], mine[d * Pp:(d + 1) * Pp])
    tri_full = torch.einsum("pik,pjk->pij", a_full, b_full)
    for r, p in enumerate(plans):
        a_r, b_r, _ = p.contract_operands(bufs[r])
        assert torch.equal(S.planes_to_dense(a_r), a_full[r * Pp:(r + 1) * Pp])
        assert torch.equal(S.planes_to_dense(b_r), b_full[r * Pp:(r + 1) * Pp])
        _, _, t_d = peer_dest_specs(p, lambda d: bufs[d]["a_recv"], lambda d: bufs[d]["b_recv"],
                                    lambda d: bufs[d]["tri_recv"])
        for d in range(world):      # rank r's planes, destination d's rows
            S.dense_to_planes(t_d[d], tri_full[r * Pp:(r + 1) * Pp, d * R:(d + 1) * R])
    for r, p in enumerate(plans):
        assert torch.equal(S.planes_to_dense(p.tri_spec(bufs[r])), tri_full[:, r * R:(r + 1) * R])


def test_peer_scheme_support_matrix():
    from miniworld_engine_b200.sharded import PeerShardContext as P
    bf16, f32 = torch.bfloat16, torch.float32
    assert P.supported(1, 2048, 128, bf16, 8)        # the benchmark configuration: 16 planes, 256 rows per rank
    assert P.supported(1, 1024, 128, bf16, 8) and P.supported(1, 512, 128, bf16, 2) and P.supported(2, 256, 128, bf16, 2)
    assert not P.supported(1, 768, 128, bf16, 8)     # 96 rows per rank: a contraction tile would straddle two ranks
    assert not P.supported(1, 2048, 128, f32, 8)     # no fp32 tensor-core kernels
    assert not P.supported(1, 2048, 64, bf16, 8)
    assert not P.supported(1, 2048, 128, bf16, 16)
    assert not P.supported(1, 1000, 128, bf16, 8)
