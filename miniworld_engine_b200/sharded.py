"""Row-sharded TriangleMultiplication block over the GPUs of one node.

Rank r owns rows ``I_r = [r*R, (r+1)*R)`` (``R = N / world``) of the pair tensor and of the
output.  Stage 1 (LayerNorm + gated projections) and stage 3 (output stage) are row-local; the
contraction couples rows, so there is exactly one exchange step per block, between stage 1 and
stage 2, done with NCCL collectives whose result the contraction kernel reads in place
(chunk-major operand planes, ``trimul_planes`` in ``include/trimul_b200.h``):

* outgoing  ``out[i,j] = sum_k a[i,k] b[j,k]``, i in I_r: ``a[I_r]`` is local, every row of ``b`` is
  needed -> **all-gather b** (row chunks: chunk s = rows I_s, produced by rank s);
* incoming  ``out[i,j] = sum_k a[k,i] b[k,j]``, i in I_r: the local z rows are the k in I_r, so
  rank r produces the k-slices ``a'[:, K_r]`` and ``b'[:, K_r]`` of the transposed operands
  (``a'[i][k] = a[k,i]``).  It needs ``a'[I_r][all k]`` -> **all-to-all of a'** (rank s sends its
  rows I_r), and ``b'[all j][all k]`` -> **all-gather b'**; both arrive as k-chunked planes.

A second exchange pattern, ``ChannelShardPlan``, moves less data: stage 1 and stage 3 stay
row-sharded, but the contraction is sharded over CHANNEL PLANES.  Each rank sends the planes it
does not own of its a and b rows to their owners (all-to-all), contracts its ``B*c/world`` planes
over the full N x N x N, and returns the rows of ``tri`` to their owners (all-to-all).  Per block
a rank receives ``3 (world-1)/world`` of one operand instead of ``(world-1)`` operand slabs.

``PeerShardContext`` runs the channel-sharded pattern WITHOUT collectives in the data path: the
three exchanges are the stores of the producing kernels themselves, aimed at the consumer
rank's memory (peer access over NVLink through symmetric-memory buffers), so the transfer of a
tile overlaps the computation of the next one and nothing is copied twice.  Only two stream-ordered
cross-GPU barriers per block remain; they are this library's own flag exchange with a bounded
wait (``trimul_b200_peer_barrier``): a rank that stopped between steps makes its peers' barrier
give up after ``barrier_timeout_us`` and report through the status words (``read_status``), which
callers of ``PeerShardContext.forward`` should poll between steps.

No k-sum is split across ranks in any pattern, so the result equals the single-GPU result.  The reference has
no distributed code at all; its single-GPU module is the behaviour to match.

The exchange logic is independent of the device: ``exchange()`` works on flat tensors with any
``torch.distributed`` backend, which is how the CPU tests drive it with gloo.
"""

from __future__ import annotations

from dataclasses import dataclass

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from . import stages as S
from .functional import _status_words

__all__ = ["ShardPlan", "ChannelShardPlan", "PeerShardContext", "peer_dest_specs", "exchange",
           "trimul_forward_sharded"]


@dataclass
class ShardPlan:
    """Sizes and operand-plane layouts of one rank's share of a block call."""

    B: int
    N: int
    c: int
    world: int
    rank: int
    outgoing: bool

    def __post_init__(self):
        if self.N % self.world != 0:
            raise ValueError(f"N={self.N} must be divisible by the number of ranks ({self.world})")
        if not 0 <= self.rank < self.world:
            raise ValueError(f"rank {self.rank} outside [0, {self.world})")
        self.R = self.N // self.world
        self.row0 = self.rank * self.R
        self.planes = self.B * self.c

    # ---- buffer sizes in elements -------------------------------------------------------
    @property
    def pitch_full(self) -> int:      # row pitch of a plane whose rows hold all N columns
        return S.round_up(self.N, 8)

    @property
    def pitch_slab(self) -> int:      # row pitch of a plane whose rows hold R columns
        return S.round_up(self.R, 8)

    def slab_elems(self) -> int:
        """Elements of one rank's contribution to a gathered operand."""
        if self.outgoing:
            return self.planes * self.R * self.pitch_full          # [P][R rows][N cols]
        return self.planes * self.N * self.pitch_slab              # [P][N rows][R cols]

    def a2a_chunk_elems(self) -> int:
        """Elements one rank sends to one peer in the incoming all-to-all: [P][R rows][R cols]."""
        return self.planes * self.R * self.pitch_slab

    # ---- plane descriptions -------------------------------------------------------------
    def tm1_outputs(self, a_buf: torch.Tensor, b_buf: torch.Tensor):
        """Where stage 1 writes.  Outgoing: ``a`` plain [P][R][N]; ``b`` straight into this rank's
        chunk of the gathered buffer.  Incoming: ``a'`` [P][N][R] row-chunked by destination rank
        (chunk r = rows I_r, contiguous, ready to be sent); ``b'`` into this rank's chunk."""
        P, R, N = self.planes, self.R, self.N
        if self.outgoing:
            a = S.PlaneSpec(a_buf, P, R, N, self.pitch_full, R * self.pitch_full)
            chunk = b_buf[self.rank * self.slab_elems():(self.rank + 1) * self.slab_elems()]
            b = S.PlaneSpec(chunk, P, R, N, self.pitch_full, R * self.pitch_full)
        else:
            a = S.PlaneSpec(a_buf, P, N, R, self.pitch_slab, R * self.pitch_slab,
                            chunk_stride=self.a2a_chunk_elems() if self.world > 1 else 0,
                            row_chunk=R if self.world > 1 else None)
            chunk = b_buf[self.rank * self.slab_elems():(self.rank + 1) * self.slab_elems()]
            b = S.PlaneSpec(chunk, P, N, R, self.pitch_slab, N * self.pitch_slab)
        return a, b

    def contract_operands(self, a_buf: torch.Tensor, b_buf: torch.Tensor):
        """How stage 2 reads the exchanged buffers.  ``a_buf`` is the local ``a`` (outgoing) or
        the all-to-all result (incoming); ``b_buf`` is the gathered operand."""
        P, R, N, W = self.planes, self.R, self.N, self.world
        if self.outgoing:
            a = S.PlaneSpec(a_buf, P, R, N, self.pitch_full, R * self.pitch_full)
            b = S.PlaneSpec(b_buf, P, N, N, self.pitch_full, R * self.pitch_full,
                            chunk_stride=self.slab_elems() if W > 1 else 0, row_chunk=R if W > 1 else None)
        else:
            a = S.PlaneSpec(a_buf, P, R, N, self.pitch_slab, R * self.pitch_slab,
                            chunk_stride=self.a2a_chunk_elems() if W > 1 else 0, col_chunk=R if W > 1 else None)
            b = S.PlaneSpec(b_buf, P, N, N, self.pitch_slab, N * self.pitch_slab,
                            chunk_stride=self.slab_elems() if W > 1 else 0, col_chunk=R if W > 1 else None)
        return a, b

    def tri_spec(self, tri_buf: torch.Tensor) -> S.PlaneSpec:
        return S.PlaneSpec(tri_buf, self.planes, self.R, self.N, self.pitch_full, self.R * self.pitch_full)

    def alloc(self, dtype: torch.dtype, device):
        """(a_send, a_recv, b_gathered, tri) buffers; ``a_recv`` is ``a_send`` when nothing moves."""
        a_elems = self.planes * self.R * self.pitch_full if self.outgoing else self.world * self.a2a_chunk_elems()
        a_send = torch.empty(a_elems, dtype=dtype, device=device)
        a_recv = a_send if (self.outgoing or self.world == 1) else torch.empty_like(a_send)
        b_full = torch.empty(self.world * self.slab_elems(), dtype=dtype, device=device)
        tri = torch.empty(self.planes * self.R * self.pitch_full, dtype=dtype, device=device)
        return a_send, a_recv, b_full, tri


def exchange(plan: ShardPlan, a_send: torch.Tensor, a_recv: torch.Tensor, b_full: torch.Tensor, group=None):
    """The block's one exchange step.  ``b_full`` already holds this rank's chunk at offset
    ``rank * slab_elems``; after the call it holds every rank's chunk.  For the incoming
    direction ``a_send`` ([world][P][R][pitch], chunk r destined for rank r) is exchanged into
    ``a_recv`` (chunk s received from rank s).  Returns the async work handles (already waited
    for backends without stream semantics)."""
    if plan.world == 1:
        return []
    n = plan.slab_elems()
    mine = b_full[plan.rank * n:(plan.rank + 1) * n]
    works = [dist.all_gather_into_tensor(b_full, mine, group=group, async_op=True)]
    if not plan.outgoing:
        works.append(dist.all_to_all_single(a_recv, a_send, group=group, async_op=True))
    for w in works:
        w.wait()
    return works


@dataclass
class ChannelShardPlan:
    """Row-sharded stage 1 / stage 3 with a channel-sharded contraction (three all-to-alls).

    Buffers (all chunk-major, chunk = peer rank, so every all-to-all moves contiguous equal
    chunks and the kernels read/write the exchanged data in place):

    * ``a_send``/``b_send``: stage 1 output in the plain plane-major layout; the planes of rank s
      are the s-th contiguous chunk;
    * ``a_recv``/``b_recv``: this rank's planes with the rows (outgoing) or the k-columns
      (incoming) of every rank: row-chunked resp. column-chunked planes;
    * ``tri_send``: contraction output for this rank's planes, row-chunked by destination rank;
    * ``tri_recv``: chunk s holds planes of rank s for this rank's rows = the plain layout.
    """

    B: int
    N: int
    c: int
    world: int
    rank: int
    outgoing: bool

    def __post_init__(self):
        if self.N % self.world != 0:
            raise ValueError(f"N={self.N} must be divisible by the number of ranks ({self.world})")
        if (self.B * self.c) % self.world != 0:
            raise ValueError(f"B*c={self.B * self.c} must be divisible by the number of ranks ({self.world})")
        if not 0 <= self.rank < self.world:
            raise ValueError(f"rank {self.rank} outside [0, {self.world})")
        self.R = self.N // self.world
        self.row0 = self.rank * self.R
        self.planes = self.B * self.c
        self.my_planes = self.planes // self.world
        self.pitch_full = S.round_up(self.N, 8)
        self.pitch_slab = S.round_up(self.R, 8)

    def _op_plane_elems(self) -> int:      # one stage-1 plane of this rank's slab
        return self.R * self.pitch_full if self.outgoing else self.N * self.pitch_slab

    def alloc(self, dtype: torch.dtype, device):
        n_op = self.planes * self._op_plane_elems()
        n_tri = self.planes * self.R * self.pitch_full
        mk = lambda n: torch.empty(n, dtype=dtype, device=device)
        return {"a_send": mk(n_op), "b_send": mk(n_op), "a_recv": mk(n_op), "b_recv": mk(n_op),
                "tri_send": mk(n_tri), "tri_recv": mk(n_tri)}

    def tm1_outputs(self, bufs):
        P, R, N = self.planes, self.R, self.N
        if self.outgoing:
            mk = lambda t: S.PlaneSpec(t, P, R, N, self.pitch_full, R * self.pitch_full)
        else:
            mk = lambda t: S.PlaneSpec(t, P, N, R, self.pitch_slab, N * self.pitch_slab)
        return mk(bufs["a_send"]), mk(bufs["b_send"])

    def contract_operands(self, bufs):
        Pp, R, N, W = self.my_planes, self.R, self.N, self.world
        if self.outgoing:   # rows of every rank: [s][Pp][R][pitch_full]
            mk = lambda t: S.PlaneSpec(t, Pp, N, N, self.pitch_full, R * self.pitch_full,
                                       chunk_stride=Pp * R * self.pitch_full if W > 1 else 0,
                                       row_chunk=R if W > 1 else None)
        else:               # k-columns of every rank: [s][Pp][N][pitch_slab]
            mk = lambda t: S.PlaneSpec(t, Pp, N, N, self.pitch_slab, N * self.pitch_slab,
                                       chunk_stride=Pp * N * self.pitch_slab if W > 1 else 0,
                                       col_chunk=R if W > 1 else None)
        tri = S.PlaneSpec(bufs["tri_send"], Pp, N, N, self.pitch_full, R * self.pitch_full,
                          chunk_stride=Pp * R * self.pitch_full if W > 1 else 0, row_chunk=R if W > 1 else None)
        return mk(bufs["a_recv"]), mk(bufs["b_recv"]), tri

    def tri_spec(self, bufs) -> S.PlaneSpec:
        return S.PlaneSpec(bufs["tri_recv"], self.planes, self.R, self.N, self.pitch_full, self.R * self.pitch_full)

    def exchange_in(self, bufs, group=None):
        if self.world == 1:
            bufs["a_recv"], bufs["b_recv"] = bufs["a_send"], bufs["b_send"]
            return
        works = [dist.all_to_all_single(bufs["a_recv"], bufs["a_send"], group=group, async_op=True),
                 dist.all_to_all_single(bufs["b_recv"], bufs["b_send"], group=group, async_op=True)]
        for w in works:
            w.wait()

    def exchange_out(self, bufs, group=None):
        if self.world == 1:
            bufs["tri_recv"] = bufs["tri_send"]
            return
        dist.all_to_all_single(bufs["tri_recv"], bufs["tri_send"], group=group)


def peer_dest_specs(cp: ChannelShardPlan, get_a, get_b, get_tri):
    """Where rank ``cp.rank`` stores what it produces, per destination rank d: its chunk inside
    d's ``a_recv`` / ``b_recv`` (stage 1 planes of d, this rank's rows) and inside d's ``tri_recv``
    (this rank's planes, d's rows).  ``get_x(d)`` returns rank d's flat receive buffer (a tensor
    whose memory this process can write: local, or a peer's through symmetric memory)."""
    Pp, R, N, r, W = cp.my_planes, cp.R, cp.N, cp.rank, cp.world
    if cp.outgoing:      # d's a_recv is [source][Pp][R][pitch_full]
        n = Pp * R * cp.pitch_full
        mk = lambda t: S.PlaneSpec(t[r * n:(r + 1) * n], Pp, R, N, cp.pitch_full, R * cp.pitch_full)
    else:                # d's a_recv is [source][Pp][N][pitch_slab]
        n = Pp * N * cp.pitch_slab
        mk = lambda t: S.PlaneSpec(t[r * n:(r + 1) * n], Pp, N, R, cp.pitch_slab, N * cp.pitch_slab)
    nt = Pp * R * cp.pitch_full      # d's tri_recv is [source][Pp][R][pitch_full]
    mt = lambda t: S.PlaneSpec(t[r * nt:(r + 1) * nt], Pp, R, N, cp.pitch_full, R * cp.pitch_full)
    return ([mk(get_a(d)) for d in range(W)], [mk(get_b(d)) for d in range(W)],
            [mt(get_tri(d)) for d in range(W)])


class PeerShardContext:
    """Buffers and peer mappings of the collective-free channel-sharded block (one per process,
    reusable for any number of calls with the same B, N, c and dtype).

    Construction is collective over ``group`` (symmetric-memory rendezvous).  ``forward`` enqueues,
    on the current stream: scattering stage 1, barrier, scattering contraction, barrier, stage 3.
    The barriers order this rank's reads after every peer's stores of the same step and keep a
    peer from overwriting a buffer that is still being read: a rank passes the first barrier of
    block t+1 only after it finished stage 3 of block t, and the second barrier of block t only
    after its contraction of block t.
    """

    @staticmethod
    def supported(B: int, N: int, c: int, dtype: torch.dtype, world: int) -> bool:
        """Whether the scattering kernels exist for this problem on ``world`` ranks: bf16, c = 128
        (tensor-core kernels), at most 8 ranks, a rank's share of the ``B*c`` planes a multiple of
        16 that divides or is a multiple of 128, and ``N/world`` rows per rank a multiple of 128.
        Otherwise use ``trimul_forward_sharded(mode="channels")``, which does the same exchanges
        with NCCL all-to-alls."""
        if dtype != torch.bfloat16 or c != 128 or not 1 <= world <= 8:
            return False
        if N % world or (B * c) % world:
            return False
        per, rows = B * c // world, N // world
        return per % 16 == 0 and (128 % per == 0 or per % 128 == 0) and rows % 128 == 0

    def __init__(self, B: int, N: int, c: int, dtype: torch.dtype, device, group=None,
                 barrier_timeout_us: int = 1_000_000):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
        import torch.distributed._symmetric_memory as symm_mem
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.B, self.N, self.c, self.dtype, self.device = B, N, c, dtype, torch.device(device)
        if not self.supported(B, N, c, dtype, self.world):
            raise ValueError(f"no scattering kernels for B={B}, N={N}, c={c}, {dtype} on {self.world} rank(s); "
                             "use trimul_forward_sharded(mode='channels')")
        plans = [ChannelShardPlan(B, N, c, self.world, self.rank, o) for o in (True, False)]
        n_op = max(p.planes * p._op_plane_elems() for p in plans)
        n_tri = plans[0].planes * plans[0].R * plans[0].pitch_full
        self._plans = {True: plans[0], False: plans[1]}
        self._local, self._handles, self._peer = {}, {}, {}
        for name, n in (("a", n_op), ("b", n_op), ("tri", n_tri)):
            t = symm_mem.empty(n, dtype=dtype, device=self.device)
            h = symm_mem.rendezvous(t, self.group)
            self._local[name], self._handles[name] = t, h
            self._peer[name] = [t if d == self.rank else h.get_buffer(d, (n,), dtype) for d in range(self.world)]
        self._dest = {o: peer_dest_specs(self._plans[o], lambda d: self._peer["a"][d], lambda d: self._peer["b"][d],
                                         lambda d: self._peer["tri"][d]) for o in (True, False)}
        # flag words of the barrier: one array of `world` int32 per rank, writable by every rank
        self.barrier_timeout_us = int(barrier_timeout_us)
        self._epoch = 0
        self._flags = symm_mem.empty(self.world, dtype=torch.int32, device=self.device)
        self._flags.zero_()
        fh = symm_mem.rendezvous(self._flags, self.group)
        self._handles["flags"] = fh
        self._flag_views = [self._flags if d == self.rank else fh.get_buffer(d, (self.world,), torch.int32)
                            for d in range(self.world)]
        self._flag_ptrs = (C.c_void_p * self.world)(*[t.data_ptr() for t in self._flag_views])
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)          # every rank's flags are zero before anyone signals

    def barrier(self) -> None:
        """Stream-ordered barrier over the ranks of the group: the library's flag exchange with a
        bounded wait.  When a peer never arrives the wait expires after ``barrier_timeout_us`` and
        the status words say so (``read_status``); nothing hangs."""
        self._epoch += 1
        st = _status_words(self.device)
        with torch.cuda.device(self.device):
            rc = _lib.load().trimul_b200_peer_barrier(
                self.rank, self.world, self._flag_ptrs, self._epoch, self.barrier_timeout_us,
                torch.cuda.current_stream(self.device).cuda_stream, st.data_ptr())
        _lib.check(rc, "trimul_b200_peer_barrier")

    @torch.no_grad()
    def forward(self, z_slab: torch.Tensor, mask, weights: dict, *, outgoing: bool, eps_in: float = 1e-5,
                eps_out: float = 1e-5, residual=None) -> torch.Tensor:
        cp = self._plans[outgoing]
        if tuple(z_slab.shape) != (self.B, cp.R, self.N, self.c) or z_slab.dtype != self.dtype:
            raise ValueError(f"slab must be {(self.B, cp.R, self.N, self.c)} {self.dtype}, got "
                             f"{tuple(z_slab.shape)} {z_slab.dtype}")
        a_dest, b_dest, tri_dest = self._dest[outgoing]
        S.tm1_scatter(z_slab, mask, weights, a_dest, b_dest, outgoing=outgoing, row0=cp.row0, eps=eps_in)
        self.barrier()
        bufs = {"a_recv": self._local["a"], "b_recv": self._local["b"], "tri_send": self._local["tri"],
                "tri_recv": self._local["tri"]}
        a_r, b_r, _ = cp.contract_operands(bufs)
        S.contract_scatter(a_r, b_r, tri_dest)
        self.barrier()
        return S.tm2(z_slab, cp.tri_spec(bufs), weights, residual=residual, row0=cp.row0,
                     eps_in=eps_in, eps_out=eps_out)


@torch.no_grad()
def trimul_forward_sharded(z_slab: torch.Tensor, mask: torch.Tensor | None, weights: dict, *, outgoing: bool,
                           N: int | None = None, group=None, eps_in: float = 1e-5, eps_out: float = 1e-5,
                           residual: torch.Tensor | None = None, buffers=None, mode: str = "rows") -> torch.Tensor:
    """One block call on this rank's ``[B, R, N, c]`` slab of the pair tensor; returns the matching
    output slab.  ``mask`` is the FULL ``[B, N]`` token mask (or ``[B, N, N]`` pair mask), identical
    on every rank.  ``weights`` is the keyword dict of ``stages.tm1`` / ``stages.tm2``.
    ``mode="rows"`` gathers the other operand (``ShardPlan``); ``mode="channels"`` shards the
    contraction over channel planes (``ChannelShardPlan``)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    B, R, Nz, c = z_slab.shape
    N = Nz if N is None else N
    if mode == "channels":
        cp = ChannelShardPlan(B, N, c, world, rank, outgoing)
        if R != cp.R:
            raise ValueError(f"slab has {R} rows, expected N/world = {cp.R}")
        bufs = buffers if buffers is not None else cp.alloc(z_slab.dtype, z_slab.device)
        a_w, b_w = cp.tm1_outputs(bufs)
        S.tm1(z_slab, mask, weights, a_w, b_w, outgoing=outgoing, row0=cp.row0, eps=eps_in)
        cp.exchange_in(bufs, group)
        a_r, b_r, tri_w = cp.contract_operands(bufs)
        S.contract(a_r, b_r, tri_w)
        cp.exchange_out(bufs, group)
        return S.tm2(z_slab, cp.tri_spec(bufs), weights, residual=residual, row0=cp.row0,
                     eps_in=eps_in, eps_out=eps_out)
    if mode != "rows":
        raise ValueError(f"mode must be rows|channels, got {mode!r}")
    plan = ShardPlan(B, N, c, world, rank, outgoing)
    if R != plan.R:
        raise ValueError(f"slab has {R} rows, expected N/world = {plan.R}")
    a_send, a_recv, b_full, tri_buf = buffers if buffers is not None else plan.alloc(z_slab.dtype, z_slab.device)
    a_w, b_w = plan.tm1_outputs(a_send, b_full)
    S.tm1(z_slab, mask, weights, a_w, b_w, outgoing=outgoing, row0=plan.row0, eps=eps_in)
    exchange(plan, a_send, a_recv, b_full, group)
    a_r, b_r = plan.contract_operands(a_recv, b_full)
    tri = plan.tri_spec(tri_buf)
    S.contract(a_r, b_r, tri)
    return S.tm2(z_slab, tri, weights, residual=residual, row0=plan.row0, eps_in=eps_in, eps_out=eps_out)
