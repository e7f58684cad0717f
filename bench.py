#!/usr/bin/env python
"""Benchmark of the B200 TriangleMultiplication block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

A step is one block call (LayerNorm_in + gated projections, contraction, LayerNorm_out +
gated output projection) on seeded synthetic input of the named workload.  Rank 0 prints
ONE JSON line:

* ``value`` / ``metric``: whole-job TFLOP/s with inputs resident in HBM, algorithmic FLOPs
  ``B*(2*N^3*c + 12*N^2*c^2)`` per call, timed with CUDA events around exactly K steps
  (barrier + synchronize on both sides, max over ranks).  Nothing is recorded between the stage
  launches of this region, so each stage is launched while its predecessor drains
  (programmatic dependent launch), as in production use;
* ``stages`` / ``roofline``: a second pass of K steps with CUDA events between the stage launches
  (which serialises them): per-stage duration, achieved rate against the measured peak in
  MEASURED_PEAKS.json; ``roofline`` is the slowest stage;
* ``e2e``: the same metric through the public module call with HOST buffers: pinned
  host->device copy of z and the mask and device->host copy of the result inside the
  timed region, every step; uploads, blocks and downloads run on three streams with two
  buffers each way (a host working through a queue), the one-stream form is reported beside it;
* ``parity_rel_rms``: relative RMS distance of the benchmarked output from the CPU oracle on
  the same seeded inputs (tolerance 1e-2 in bf16);
* ``comparators``: ``torch.bmm`` (cuBLAS) on the very operand planes the contraction reads, timed
  the same way — the kernel the reference's contraction lands on;
* ``cpu_baseline``: the CPU oracle (a port of the reference's reference.py) timed on this
  box's host cores on a bounded sample (rank 0, N=1 only);
* ``clocks``: SM clock and throttle reasons sampled through NVML while all timed legs run.

Workloads
  n768_outgoing (default)  bf16, B=1, N=768, c=128, all-ones token mask: the configuration
                           the headline metric is quoted on.  With --gpus N > 1 every rank
                           runs its own block on its own pair tensor (weak scaling, no
                           collective in the data path: independent pair tensors), and the line
                           carries a ``sharded_n2048`` record beside it: BASELINE config 5 with the
                           output rows sharded over the N ranks (strong scaling), its speed-up over
                           one GPU measured in the same run and a bit-for-bit comparison of every
                           rank's slab with the unsharded result.
  n384_outgoing            BASELINE config 2.
  n768_incoming_pad77      BASELINE config 3.
  n512_b2_outgoing_c64/c256, n384_outgoing_c256
                           BASELINE config 4 (d_pair sweep) and the reference's published c=256 case.
  n2048_pair_sharded       BASELINE config 5: outgoing then incoming block at N=2048, output rows
                           sharded over the ranks (strong scaling, one exchange per block).

``--impl reference`` times the CPU oracle on the host cores instead (rank 0 only).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, N, c, outgoing, mask kind)
    "n768_outgoing": (1, 768, 128, True, "ones"),
    "n384_outgoing": (1, 384, 128, True, "ones"),
    "n768_incoming_pad77": (1, 768, 128, False, "tail77"),
    "n1024_outgoing": (1, 1024, 128, True, "ones"),
    "n2048_outgoing": (1, 2048, 128, True, "rand5"),
    # other channel widths (BASELINE config 4 and the reference's d_pair sweep): stages 1 and 3 run on
    # the warp-MMA kernels there, the contraction on the same tcgen05 kernel
    "n384_outgoing_c256": (1, 384, 256, True, "ones"),
    "n512_b2_outgoing_c256": (2, 512, 256, True, "ones"),
    "n512_b2_outgoing_c64": (2, 512, 64, True, "ones"),
}
# The bidirectional block (outgoing contraction on the first 128 hidden channels, incoming on the
# second 128, one LayerNorm over all 256, residual added): single GPU, stage split by CUDA events.
BIDIR_WORKLOADS = {
    "n768_bidirectional": (1, 768, 128, "ones"),
    "n512_bidirectional": (1, 512, 128, "ones"),
    "n384_bidirectional": (1, 384, 128, "ones"),
}
# Outgoing block then incoming block on its output, output rows sharded over the ranks
# (BASELINE config 5 at N=2048; the smaller ones are quick checks).  Strong scaling.
PAIR_WORKLOADS = {
    "n2048_pair_sharded": (1, 2048, 128, "rand5"),
    "n1024_pair_sharded": (1, 1024, 128, "rand5"),
    "n512_pair_sharded": (1, 512, 128, "rand5"),
}
METRIC = "trimul_block_tflops"
UNIT = "TFLOP/s"
# The reference publishes this metric on a B200 for its own sm_100 path, module forward (block +
# residual add), bf16, B=1, c=128, measured by CUDA-graph replay: 0.5437 ms at N=768 = 427 TFLOP/s
# with the FLOP count used here, 0.1596 ms at N=384, 0.9891 ms at N=1024
# (benchmarks/modules/triangle_multiplication/results/b200/tables/inference_seq_len.csv:17,5,25), and
# 0.3072 ms at N=384 with c=256 (.../inference_d_pair.csv:9).
PUBLISHED_MS = {"n768_outgoing": 0.5437, "n384_outgoing": 0.1596, "n1024_outgoing": 0.9891,
                "n384_outgoing_c256": 0.3072}
PUBLISHED_TFLOPS = {k: WORKLOADS[k][0] * (2.0 * WORKLOADS[k][1] ** 3 * WORKLOADS[k][2] +
                                          12.0 * WORKLOADS[k][1] ** 2 * WORKLOADS[k][2] ** 2) / (ms * 1e-3) / 1e12
                    for k, ms in PUBLISHED_MS.items()}
# DRAM bytes per launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum) on the
# n768_outgoing workload, as multiples of S = B*N*N*c*2 bytes; other sizes are scaled by S
# (all three kernels stream their operands once, so traffic grows in proportion).
NCU_TRAFFIC_PER_S = {"tm1": 2.62, "contract": 2.81, "tm2": 2.77}
# c = 256 kernels: captured at N=384 only (profiles/ncu_full_n384_c256_wide_stage1_stage3.md), where
# part of the operands stay in L2 between the stages, so these bytes are quoted for that workload only
NCU_TRAFFIC_BYTES = {"n384_outgoing_c256": {"tm1": 169.6e6, "contract": None, "tm2": 193.1e6}}


def block_flops(B, N, c):
    return float(B) * (2.0 * N ** 3 * c + 12.0 * N ** 2 * c ** 2)


def workload_config(name, B, N, c, direction, mask_kind):
    """The ``config`` object of a workload: identical in both arms (b200 and reference)."""
    S_mb = B * N * N * c * 2 / 1e6
    return {"workload": name, "B": B, "N": N, "c": c, "direction": direction, "mask": mask_kind,
            "l2": ("working set 5 x %.0f MB per call exceeds the 126 MB L2; no flush" % S_mb if 5 * S_mb > 126 else
                   "working set 5 x %.0f MB per call fits the 126 MB L2: stages chain through L2, as in the "
                   "reference's own measurement; no flush" % S_mb)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML (read-only queries) from a
    background thread while the timed region runs."""

    def __init__(self, gpu_index: int, period_s: float = 0.005):
        import threading
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            # NVML indexes physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    phys = int(ids[gpu_index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None
            return
        self._period = period_s
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nv
        names = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"),
                 ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
                 ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"),
                 ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap"))
        alt = {"nvmlClocksEventReasonHwSlowdown": "nvmlClocksThrottleReasonHwSlowdown",
               "nvmlClocksEventReasonHwThermalSlowdown": "nvmlClocksThrottleReasonHwThermalSlowdown",
               "nvmlClocksEventReasonSwThermalSlowdown": "nvmlClocksThrottleReasonSwThermalSlowdown",
               "nvmlClocksEventReasonSwPowerCap": "nvmlClocksThrottleReasonSwPowerCap"}
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                if get_reasons is not None:
                    r = get_reasons(self._h)
                    for label, const in names:
                        bit = getattr(nv, const, None) or getattr(nv, alt[const], 0)
                        if r & bit:
                            self.reasons.add(label)
            except Exception:
                pass
            time.sleep(self._period)

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        if self._thread is None:
            return out
        self._stop.set()
        self._thread.join(timeout=2)
        if self.samples:
            out.update(sm_mhz=statistics.median(self.samples), reasons=sorted(self.reasons),
                       samples=len(self.samples))
        return out


def cpu_oracle_rate(B, N, c, outgoing, mask_kind, budget_s=25.0, max_calls=3):
    """TFLOP/s of the CPU oracle on this host, all cores, bf16 like the GPU workload."""
    import torch
    from oracle import trimul_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = O.make_weights(c, 0).to(torch.bfloat16)
    z = O.make_input(B, N, c, 1).to(torch.bfloat16)
    m = O.make_token_mask(B, N, mask_kind)
    t0 = time.perf_counter()
    O.trimul_forward(z, m, w, outgoing)                      # warm-up (thread pools, allocator)
    warm = time.perf_counter() - t0
    best, calls, y = float("inf"), 0, None
    while calls < max_calls and (calls == 0 or (time.perf_counter() - t0) + best < budget_s):
        t1 = time.perf_counter()
        y = O.trimul_forward(z, m, w, outgoing)
        best = min(best, time.perf_counter() - t1)
        calls += 1
    return {"value": block_flops(B, N, c) / best / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "seconds_per_call": best,
            "sample": f"{calls} full block call(s) of the same workload (bf16 oracle, best of {calls}, "
                      f"warm-up {warm:.2f}s)"}, y


def run_reference(args):
    """Reference arm: the reference's CPU algorithm (oracle port) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import trimul_oracle as O
    pair = args.workload in PAIR_WORKLOADS
    if pair:
        B, N, c, mask_kind = PAIR_WORKLOADS[args.workload]
        outgoing = True
    else:
        B, N, c, outgoing, mask_kind = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = O.make_weights(c, 0).to(torch.bfloat16)
    w2 = O.make_weights(c, 3).to(torch.bfloat16)
    z = O.make_input(B, N, c, 1).to(torch.bfloat16)
    m = O.make_token_mask(B, N, mask_kind)

    def call():
        y = O.trimul_forward(z, m, w, outgoing)
        if pair:
            y = O.trimul_forward(y, m, w2, False)
        return y

    for _ in range(args.warmup):
        call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call()
    dt = time.perf_counter() - t0
    val = (2.0 if pair else 1.0) * block_flops(B, N, c) * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "calls_per_s": args.steps / dt, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded randn, all on the host)",
        "config": workload_config(args.workload, B, N, c,
                                  "outgoing then incoming" if pair else ("outgoing" if outgoing else "incoming"),
                                  mask_kind),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full block calls per run (each step = one call of the workload)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_b200(args):
    import torch
    import torch.distributed as dist
    from oracle import trimul_oracle as O
    from miniworld_engine_b200 import TriangleMultiplicationB200, read_status, stages as S

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the b200 arm has no CPU path (use --impl reference)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # stdout carries the one JSON line and nothing else: the collective library's own messages
        # (its version banner, anything NCCL_DEBUG asks for) go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    B, N, c, outgoing, mask_kind = WORKLOADS[args.workload]
    flops = block_flops(B, N, c)
    # synthetic inputs: weights seed 0, input seed 1 (+rank: every rank its own pair tensor)
    w = O.make_weights(c, 0)
    z_host = O.make_input(B, N, c, 1 + rank).to(torch.bfloat16).pin_memory()
    m_host = O.make_token_mask(B, N, mask_kind).pin_memory()
    mod = TriangleMultiplicationB200(c, outgoing=outgoing)
    mod.load_state_dict(w.state_dict())
    mod = mod.to(dev).to(torch.bfloat16).eval()
    z = z_host.to(dev)
    m = m_host.to(dev)
    wd = dict(ln_in_w=mod.ln_pair.weight, ln_in_b=mod.ln_pair.bias, w_left=mod.to_left.weight,
              w_left_gate=mod.to_left_gate.weight, w_right=mod.to_right.weight,
              w_right_gate=mod.to_right_gate.weight, ln_out_w=mod.ln_out.weight, ln_out_b=mod.ln_out.bias,
              w_gate=mod.to_gate.weight, w_out=mod.to_out.weight)
    planes = B * c
    a = S.alloc_planes(planes, N, N, torch.bfloat16, dev)
    b = S.alloc_planes(planes, N, N, torch.bfloat16, dev)
    tri = S.alloc_planes(planes, N, N, torch.bfloat16, dev)

    def step(ev=None, residual=None):
        """One block call = the three stage launches of trimul_b200_forward, with optional
        events between them."""
        if ev is not None:
            ev[0].record()
        S.tm1(z, m, wd, a, b, outgoing=outgoing)
        if ev is not None:
            ev[1].record()
        S.contract(a, b, tri)
        if ev is not None:
            ev[2].record()
        out = S.tm2(z, tri, wd, residual=residual)
        if ev is not None:
            ev[3].record()
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, n):
        """n calls of fn between two events; nothing recorded in between."""
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        barrier()
        return t0.elapsed_time(t1)

    # the clock sampler and the first collective (communicator set-up) start BEFORE the warm-up steps, so
    # that their start-up cost on the host — on an 8-GPU node it was seen to double the first timed
    # region of a short run — falls into the warm-up and not into the timed region
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # the timed region: exactly K steps, stages launched back to back
    total_ms = timed(step, args.steps)
    rank_ms = None
    if world > 1:      # every rank's own figure beside the maximum, so that a straggler shows
        g = [torch.zeros(1, device=dev, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(g, torch.tensor([total_ms / args.steps], device=dev, dtype=torch.float64))
        rank_ms = [float(v) for v in torch.cat(g).cpu()]
    # the same K steps again with events between the stages (per-stage durations for the roofline)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    barrier()
    for k in range(args.steps):
        step(evs[k])
    barrier()
    staged_ms = evs[0][0].elapsed_time(evs[-1][3]) / args.steps
    stage_ms = [sum(e[i].elapsed_time(e[i + 1]) for e in evs) / args.steps for i in range(3)]
    st = read_status(dev)
    if st[0] != 0:
        raise SystemExit(f"bench.py: device status {st}: a bounded wait expired, timing is invalid")

    # each stage once more by itself: an L2 flush (a 256 MB fill) before every launch, which is also a
    # pause — kernels repeated without one run 10-18 % slower on this part, as the sustained GEMM peak
    # sits below the burst peak; the in-step durations above are what the roofline line uses
    alone_ms = None
    if rank == 0:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        calls = (lambda: S.tm1(z, m, wd, a, b, outgoing=outgoing), lambda: S.contract(a, b, tri),
                 lambda: S.tm2(z, tri, wd))
        alone_ms = []
        n_alone = max(5, min(args.steps, 20))
        for fn in calls:
            fn()                      # (a variant without the residual may not have run yet: module load)
            tot = 0.0
            for _ in range(n_alone):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize(dev)
                tot += e0.elapsed_time(e1)
            alone_ms.append(tot / n_alone)
        del flush

    # the same step with the residual fused into the output stage (what the reference MODULE returns)
    step_res = lambda: step(residual=z)
    for _ in range(3):
        step_res()
    res_ms = timed(step_res, args.steps) / args.steps

    # the same step (residual fused) captured once in a CUDA graph and replayed: no host work per
    # step, which is how the reference's published table was measured (cudagraph=manual)
    graph = torch.cuda.CUDAGraph()
    # thread_local: another thread of this process (a collective library's watchdog) may touch the
    # CUDA API while this thread captures
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        y_graph = step_res()
    for _ in range(3):
        graph.replay()
    graph_ms = timed(graph.replay, args.steps) / args.steps
    if not torch.equal(y_graph, step_res()):
        raise SystemExit("bench.py: the CUDA-graph replay and the eager step disagree")
    del graph, y_graph

    # comparator: cuBLAS (torch.bmm) on the very planes the contraction reads — the kernel the
    # reference's contraction lands on (module.py:439-442); same events, same warm-up
    comparators = None
    if a.pitch == N and rank == 0:
        a3 = a.buf[: planes * a.plane_stride].view(planes, N, N)
        b3 = b.buf[: planes * b.plane_stride].view(planes, N, N)
        t3 = torch.empty(planes, N, N, dtype=torch.bfloat16, device=dev)
        bmm = lambda: torch.bmm(a3, b3.transpose(1, 2), out=t3)
        for _ in range(3):
            bmm()
        torch.cuda.synchronize(dev)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(args.steps):
            bmm()
        c1.record()
        torch.cuda.synchronize(dev)
        bmm_ms = c0.elapsed_time(c1) / args.steps
        S.contract(a, b, tri)
        own = S.planes_to_dense(tri)
        comparators = {"cublas_bmm_ms": bmm_ms, "cublas_bmm_tflops": 2.0 * B * N ** 3 * c / (bmm_ms * 1e-3) / 1e12,
                       "contract_ms": stage_ms[1],
                       "contract_vs_cublas_rel_rms": float((own.float() - t3.float()).norm() / t3.float().norm()),
                       "what": "torch.bmm(a, b^T) over the same B*c operand planes, device-timed back to back"}
        del t3, own

    # end to end through the public module call, host buffers in and out.  Every step copies its
    # input from pinned host memory and its result back to pinned host memory; as a host that
    # works through a queue of pair tensors would, the copies run on their own streams with two
    # buffers each way, so the upload of step i+1 and the download of step i-1 overlap the block
    # of step i (PCIe is full duplex).  The serial form (one stream) is reported beside it.
    out_host = [torch.empty(z_host.shape, dtype=z_host.dtype).pin_memory() for _ in range(2)]
    zd = [torch.empty_like(z) for _ in range(2)]
    md = [torch.empty_like(m) for _ in range(2)]
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_run(n):
        torch.cuda.synchronize(dev)
        ev_in = [None, None]; ev_cmp = [None, None]; ev_out = [None, None]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(s_in)
        for i in range(n):
            k = i & 1
            with torch.cuda.stream(s_in):
                if ev_cmp[k] is not None:
                    s_in.wait_event(ev_cmp[k])            # the block two steps ago has read zd[k]
                zd[k].copy_(z_host, non_blocking=True)
                md[k].copy_(m_host, non_blocking=True)
                ev_in[k] = torch.cuda.Event(); ev_in[k].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[k])
                y = mod.block(zd[k], md[k])
                ev_cmp[k] = torch.cuda.Event(); ev_cmp[k].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[k])
                out_host[k].copy_(y, non_blocking=True)   # (a queue consumer would take out_host[k] after ev_out[k])
                y.record_stream(s_out)
                ev_out[k] = torch.cuda.Event(); ev_out[k].record(s_out)
        s_out.wait_stream(s_in)
        s_out.wait_stream(s_cmp)
        t1.record(s_out)
        torch.cuda.synchronize(dev)
        return t0.elapsed_time(t1) / n

    def e2e_serial(n):
        torch.cuda.synchronize(dev)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            zd[0].copy_(z_host, non_blocking=True)
            md[0].copy_(m_host, non_blocking=True)
            y = mod.block(zd[0], md[0])
            out_host[0].copy_(y, non_blocking=True)
        t1.record()
        torch.cuda.synchronize(dev)
        return t0.elapsed_time(t1) / n

    e2e_steps = max(4, min(args.steps, 12))
    e2e_run(2)
    barrier()
    # the host link is shared with the machine's other tenants: two passes, the quieter one counts
    e2e_pipelined_ms = min(e2e_run(e2e_steps), e2e_run(e2e_steps))
    barrier()
    e2e_serial_ms = e2e_serial(max(3, e2e_steps // 2))
    barrier()
    e2e_ms = min(e2e_pipelined_ms, e2e_serial_ms)
    e2e_how = ("pinned host buffers, upload / block / download on three streams, two buffers each way"
               if e2e_pipelined_ms <= e2e_serial_ms else
               "pinned host buffers, upload, block and download in order on one stream (the three-stream "
               "form was slower on this host)")
    if not torch.equal(out_host[0], out_host[1]):
        raise SystemExit("bench.py: the two end-to-end result buffers differ")

    clocks = sampler.stop() if sampler else None
    t = torch.tensor([total_ms, e2e_ms, res_ms, graph_ms, staged_ms] + stage_ms, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, res_ms, graph_ms, staged_ms, *stage_ms = [float(v) for v in t.cpu()]

    # the benchmarked output itself, for the comparison with the oracle further down
    y_dev = step().float().cpu() if (rank == 0 and not args.no_cpu_baseline) else None

    # BASELINE config 5 beside the replica line: rows sharded over the ranks, checked bit for bit
    sharded = None
    if world > 1:
        del a, b, tri
        torch.cuda.empty_cache()
        sharded = measure_sharded_pair("n2048_pair_sharded", "auto", max(5, min(args.steps, 10)), 3, dev, rank, world,
                                       check=True, one_gpu=True)

    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = total_ms / args.steps
        value = flops * world / (ms_per_step * 1e-3) / 1e12
        S_bytes = B * N * N * c * 2
        stage_info = {
            "tm1": {"ms": stage_ms[0], "bound": "hbm", "achieved": 3 * S_bytes / (stage_ms[0] * 1e-3) / 1e9,
                    "unit": "GB/s", "peak": peaks["hbm_gbs"]},
            "contract": {"ms": stage_ms[1], "bound": "tensor",
                         "achieved": 2.0 * B * N ** 3 * c / (stage_ms[1] * 1e-3) / 1e12, "unit": "TFLOP/s",
                         "peak": peaks["bf16_tflops"], "frac_of_sustained": None},
            "tm2": {"ms": stage_ms[2], "bound": "hbm", "achieved": 3 * S_bytes / (stage_ms[2] * 1e-3) / 1e9,
                    "unit": "GB/s", "peak": peaks["hbm_gbs"]},
        }
        stage_info["contract"]["frac_of_sustained"] = stage_info["contract"]["achieved"] / peaks["bf16_tflops_sustained"]
        for i, (k, v) in enumerate(stage_info.items()):
            v["frac"] = v["achieved"] / v["peak"]
            if alone_ms is not None:      # the same launch by itself after an L2 flush
                v["ms_alone"] = alone_ms[i]
                v["frac_alone"] = v["frac"] * v["ms"] / alone_ms[i]
            # bytes per launch, from the ncu capture of the c = 128 kernels (none for the other widths)
            v["traffic"] = (NCU_TRAFFIC_PER_S[k] * S_bytes if c == 128 else
                            NCU_TRAFFIC_BYTES.get(args.workload, {}).get(k))
        dom = max(stage_info, key=lambda k: stage_info[k]["ms"])
        roof = dict(stage_info[dom])
        roof.update(kernel=dom, peak_source=peaks["source"],
                    algorithmic=(3 * S_bytes if roof["bound"] == "hbm" else 2.0 * B * N ** 3 * c),
                    algorithmic_unit="bytes" if roof["bound"] == "hbm" else "flop",
                    how="stage durations from the pass with CUDA events between the stage launches "
                        f"({staged_ms:.4f} ms per step against {ms_per_step:.4f} ms without the events)")
        config = workload_config(args.workload, B, N, c, "outgoing" if outgoing else "incoming", mask_kind)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "calls_per_s": world * 1e3 / ms_per_step,
            "higher_is_better": True, "scaling": "weak",
            # against the reference's published module number, which includes the residual add:
            # compare like with like (our step with the fused residual), per GPU
            "vs_baseline": (flops / (res_ms * 1e-3) / 1e12 / PUBLISHED_TFLOPS[args.workload]
                            if args.workload in PUBLISHED_TFLOPS else None),
            "with_residual": {"ms_per_step": res_ms, "value": flops * world / (res_ms * 1e-3) / 1e12, "unit": UNIT},
            "cuda_graph_replay": {"ms_per_step": graph_ms, "value": flops * world / (graph_ms * 1e-3) / 1e12,
                                  "unit": UNIT, "what": "the with_residual step captured once and replayed"},
            "staged_ms_per_step": staged_ms,
            "rank_ms_per_step": rank_ms,
            "dtype": "bf16",
            "data": "synthetic (seeded randn pair tensor and weights, all-ones LayerNorm gamma)",
            "frac_of_bf16_peak": value / world / peaks["bf16_tflops"],
            "config": config,
            "parallelism": "one block per GPU, no collective" if world > 1 else "single GPU",
            "gpu_launches": 3 * args.steps,
            "e2e": {"value": flops * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "pipelined_ms_per_step": e2e_pipelined_ms, "serial_ms_per_step": e2e_serial_ms,
                    "how": e2e_how,
                    "h2d_bytes_per_step": z_host.numel() * 2 + m_host.numel(),
                    "d2h_bytes_per_step": out_host[0].numel() * 2},
            "roofline": roof, "stages": stage_info, "comparators": comparators, "clocks": clocks,
        }
        if sharded is not None:
            line["sharded_n2048"] = sharded
        if not args.no_cpu_baseline:
            # the oracle call also gives the reference output for this very input: parity of the
            # benchmarked kernels (rank 0's pair tensor is seed 1, the oracle's)
            base, y_ref = cpu_oracle_rate(B, N, c, outgoing, mask_kind, budget_s=25.0 if world == 1 else 5.0,
                                          max_calls=3 if world == 1 else 1)
            if world == 1:
                line["cpu_baseline"] = base
            line["parity_rel_rms"] = O.rel_rms(y_dev, y_ref.float())
            line["parity_tolerance"] = 1e-2
            if not line["parity_rel_rms"] <= 1e-2:
                raise SystemExit(f"bench.py: parity against the oracle failed: rel-RMS {line['parity_rel_rms']:.3e}")
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_sharded_pair(workload, shard_mode, steps, warmup, dev, rank, world, *, check=True, one_gpu=False):
    """Outgoing block followed by an incoming block on its output (independent weight sets, seeds 0
    and 3), rows sharded over the ranks; the process group must already exist when world > 1.

    ``shard_mode``: "rows" (NCCL all-gather of b, all-to-all of a for the incoming block),
    "channels" (three NCCL all-to-alls per block), "peer" (no collective: the producing kernels store
    into the consumer GPU's memory, two bounded flag barriers per block) or "auto" (peer where its
    kernels exist for the problem, else channels).  ``check``: every rank also computes the unsharded
    pair on its own GPU and compares its slab with it, bit for bit.  ``one_gpu``: that unsharded pair
    is timed on rank 0 and the speed-up over it reported.  Returns the record on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist
    from oracle import trimul_oracle as O
    from miniworld_engine_b200 import read_status, stages as S, trimul_forward
    from miniworld_engine_b200.sharded import ChannelShardPlan, PeerShardContext, ShardPlan, exchange

    B, N, c, mask_kind = PAIR_WORKLOADS[workload]
    if shard_mode == "auto":
        shard_mode = "peer" if (world > 1 and PeerShardContext.supported(B, N, c, torch.bfloat16, world)) else "channels"
    R = N // world
    g = torch.Generator().manual_seed(1)
    slabs = []
    for r in range(world):      # the same seeded tensor on every rank, generated slab by slab
        blk = torch.randn(B, R, N, c, generator=g).to(torch.bfloat16)
        if r == rank or check:
            slabs.append(blk.to(dev))
        if r == rank:
            z_slab = slabs[-1]
    m = O.make_token_mask(B, N, mask_kind).to(dev)

    def wdict(seed):
        w = O.make_weights(c, seed).to(torch.bfloat16)
        return dict(ln_in_w=w.ln_pair_weight.to(dev), ln_in_b=w.ln_pair_bias.to(dev), w_left=w.to_left.to(dev),
                    w_left_gate=w.to_left_gate.to(dev), w_right=w.to_right.to(dev),
                    w_right_gate=w.to_right_gate.to(dev), ln_out_w=w.ln_out_weight.to(dev),
                    ln_out_b=w.ln_out_bias.to(dev), w_gate=w.to_gate.to(dev), w_out=w.to_out.to(dev))

    w_out, w_in = wdict(0), wdict(3)
    peer = shard_mode == "peer"
    channels = shard_mode == "channels" or peer
    Plan = ChannelShardPlan if channels else ShardPlan
    plans = {True: Plan(B, N, c, world, rank, True), False: Plan(B, N, c, world, rank, False)}
    if peer:
        ctx = PeerShardContext(B, N, c, torch.bfloat16, dev)
        bufs = {k: {"a_recv": ctx._local["a"], "b_recv": ctx._local["b"], "tri_send": ctx._local["tri"],
                    "tri_recv": ctx._local["tri"]} for k in plans}
    else:
        bufs = {k: p.alloc(torch.bfloat16, dev) for k, p in plans.items()}

    def mark(ev):
        ev.append(torch.cuda.Event(enable_timing=True))
        ev[-1].record()

    def block_channels(x, wd, outgoing, ev):
        p, bf = plans[outgoing], bufs[outgoing]
        a_w, b_w = p.tm1_outputs(bf)
        S.tm1(x, m, wd, a_w, b_w, outgoing=outgoing, row0=p.row0)
        mark(ev)
        p.exchange_in(bf)
        a_r, b_r, tri_w = p.contract_operands(bf)
        S.contract(a_r, b_r, tri_w)
        mark(ev)            # "exchange" slot = all-to-all in + contraction start; see stage names below
        p.exchange_out(bf)
        mark(ev)
        y = S.tm2(x, p.tri_spec(bf), wd, row0=p.row0)
        mark(ev)
        return y

    def block_peer(x, wd, outgoing, ev):
        # the exchanges are the stores of the scattering kernels; only barriers stand between stages
        p, bf = plans[outgoing], bufs[outgoing]
        a_dest, b_dest, tri_dest = ctx._dest[outgoing]
        S.tm1_scatter(x, m, wd, a_dest, b_dest, outgoing=outgoing, row0=p.row0)
        mark(ev)
        ctx.barrier()
        a_r, b_r, _ = p.contract_operands(bf)
        S.contract_scatter(a_r, b_r, tri_dest)
        mark(ev)
        ctx.barrier()
        mark(ev)
        y = S.tm2(x, p.tri_spec(bf), wd, row0=p.row0)
        mark(ev)
        return y

    def block(x, wd, outgoing, ev):
        if peer:
            return block_peer(x, wd, outgoing, ev)
        if channels:
            return block_channels(x, wd, outgoing, ev)
        p = plans[outgoing]
        a_send, a_recv, b_full, tri_buf = bufs[outgoing]
        a_w, b_w = p.tm1_outputs(a_send, b_full)
        S.tm1(x, m, wd, a_w, b_w, outgoing=outgoing, row0=p.row0)
        mark(ev)
        exchange(p, a_send, a_recv, b_full)
        mark(ev)
        a_r, b_r = p.contract_operands(a_recv, b_full)
        tri = p.tri_spec(tri_buf)
        S.contract(a_r, b_r, tri)
        mark(ev)
        y = S.tm2(x, tri, wd, row0=p.row0)
        mark(ev)
        return y

    def step():
        ev = [torch.cuda.Event(enable_timing=True)]
        ev[0].record()
        y1 = block(z_slab, w_out, True, ev)
        y2 = block(y1, w_in, False, ev)
        return ev, y2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(dev.index) if rank == 0 else None
    barrier()
    all_ev = [step()[0] for _ in range(steps)]
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = all_ev[0][0].elapsed_time(all_ev[-1][-1])
    names = (["tm1+scatter", "barrier+contract+scatter", "barrier", "tm2"] if peer else
             ["tm1", "a2a_in+contract", "a2a_out", "tm2"] if channels else ["tm1", "exchange", "contract", "tm2"])
    stage_ms = [sum(e[i].elapsed_time(e[i + 1]) + e[i + 4].elapsed_time(e[i + 5]) for e in all_ev) / steps
                for i in range(4)]
    if read_status(dev)[0] != 0:
        raise SystemExit(f"bench.py: device status {read_status(dev)}: timing is invalid")

    # every rank: the unsharded pair on its own GPU (same kernels through the public functional op)
    parity, one_gpu_ms = None, None
    if check:
        y_slab = step()[1]
        z_full = torch.cat(slabs, dim=1)
        del slabs

        def kw(wd):
            return dict(ln_in_weight=wd["ln_in_w"], ln_in_bias=wd["ln_in_b"], w_left=wd["w_left"],
                        w_left_gate=wd["w_left_gate"], w_right=wd["w_right"], w_right_gate=wd["w_right_gate"],
                        ln_out_weight=wd["ln_out_w"], ln_out_bias=wd["ln_out_b"], w_gate=wd["w_gate"], w_out=wd["w_out"])

        def whole():
            y1 = trimul_forward(z_full, m, outgoing=True, **kw(w_out))
            return trimul_forward(y1, m, outgoing=False, **kw(w_in))

        y_full = whole()
        mine = y_full[:, rank * R:(rank + 1) * R]
        bit = bool(torch.equal(y_slab, mine))
        rel = float((y_slab.float() - mine.float()).norm() / mine.float().norm())
        del y_full, mine
        if one_gpu:
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                whole()
            e1.record()
            torch.cuda.synchronize(dev)
            one_gpu_ms = e0.elapsed_time(e1) / 3
        flags = torch.tensor([1.0 if bit else 0.0, -rel], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        parity = {"bit_identical": bool(flags[0].item() == 1.0), "rel_rms_vs_unsharded": float(-flags[1].item()),
                  "what": "every rank's output slab against the unsharded pair of blocks computed on the same GPU"}
        if read_status(dev)[0] != 0:
            raise SystemExit(f"bench.py: device status {read_status(dev)} after the unsharded check")
        if not parity["rel_rms_vs_unsharded"] <= 1e-2:
            raise SystemExit(f"bench.py: sharded result differs from the unsharded one: {parity}")

    t = torch.tensor([total_ms] + stage_ms + [one_gpu_ms if (one_gpu_ms is not None and rank == 0) else 0.0],
                     device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, *stage_ms, one_gpu_ms = [float(v) for v in t.cpu()]
    if rank != 0:
        return None
    peaks = measured_peaks()
    flops = 2.0 * block_flops(B, N, c)
    ms = total_ms / steps
    gathered = (world - 1) * R * N * c * 2 * B          # bytes each rank receives per all-gather
    a2a = (world - 1) * R * R * c * 2 * B               # and in the incoming all-to-all
    if channels:                                        # three exchanges of (world-1)/world slabs
        gathered, a2a = 3 * (world - 1) * R * N * (c // world) * 2 * B, 0
    rec = {
        "workload": workload, "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT,
        "calls_per_s": 2e3 / ms, "steps": steps, "scaling": "strong", "shard_mode": shard_mode,
        "frac_of_bf16_peak": flops / (ms * 1e-3) / 1e12 / world / peaks["bf16_tflops"],
        "parallelism": (f"rows sharded over {world} GPU(s), contraction sharded over channel planes, "
                        "exchanges done by the kernels' own stores into peer memory, two bounded flag barriers per block")
        if peer else (f"rows sharded over {world} GPU(s), contraction sharded over channel planes, "
                      "three all-to-alls per block") if channels else
        (f"output rows sharded over {world} GPU(s), all-gather of b per block, "
         "all-to-all of a for the incoming block"),
        "nvlink_bytes_received_per_rank_per_step": 2 * gathered + a2a,
        "stages": {n: {"ms": v} for n, v in zip(names, stage_ms)},
        "gpu_launches": (10 if peer else 6) * steps,
        "clocks": clocks,
    }
    if parity is not None:
        rec["sharded_parity"] = parity
    if one_gpu and one_gpu_ms > 0:
        rec["one_gpu_ms_per_step"] = one_gpu_ms
        rec["speedup_over_one_gpu"] = one_gpu_ms / ms
    return rec


def run_sharded_pair(args):
    """BASELINE config 5 as the line's own workload (``--workload n2048_pair_sharded``)."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the b200 arm has no CPU path (use --impl reference)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # stdout carries the one JSON line and nothing else: the collective library's own messages
        # (its version banner, anything NCCL_DEBUG asks for) go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    elif args.shard_mode == "peer":
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1, device_id=dev)
    rec = measure_sharded_pair(args.workload, args.shard_mode, args.steps, args.warmup, dev, rank, world,
                               check=not args.no_check, one_gpu=world > 1)
    if rank == 0:
        B, N, c, mask_kind = PAIR_WORKLOADS[args.workload]
        line = {
            "metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "calls_per_s": rec["calls_per_s"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded randn pair tensor and weights)",
            "frac_of_bf16_peak": rec["frac_of_bf16_peak"],
            "config": workload_config(args.workload, B, N, c, "outgoing then incoming", mask_kind),
            "parallelism": rec["parallelism"],
        }
        for k in ("shard_mode", "nvlink_bytes_received_per_rank_per_step", "gpu_launches", "stages", "clocks",
                  "sharded_parity", "one_gpu_ms_per_step", "speedup_over_one_gpu"):
            if k in rec:
                line[k] = rec[k]
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def run_bidirectional(args):
    """One bidirectional block per step on one GPU (the reference's pair-track variant,
    modules/triangle_multiplication/bidirectional.py:93-156), inputs resident in HBM."""
    import torch
    from oracle import trimul_oracle as O
    from miniworld_engine_b200 import read_status, stages as S

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the b200 arm has no CPU path (use --impl reference)")
    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("bench.py: the bidirectional workloads are single-GPU")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, N, d, mask_kind = BIDIR_WORKLOADS[args.workload]
    h = d
    w = O.make_bidir_weights(d, h, 0).to(torch.bfloat16)
    z = O.make_input(B, N, d, 1).to(torch.bfloat16).to(dev)
    m = O.make_token_mask(B, N, mask_kind).to(dev)
    t = lambda x: x.to(dev)
    ln_in = (t(w.ln_pair_weight), t(w.ln_pair_bias))
    wl, wlg, wr, wrg = t(w.to_left), t(w.to_left_gate), t(w.to_right), t(w.to_right_gate)
    w_gate, w_out = t(w.to_gate), t(w.to_out)
    planes = B * 2 * h
    a = S.alloc_planes(planes, N, N, torch.bfloat16, dev)
    b = S.alloc_planes(planes, N, N, torch.bfloat16, dev)
    tri = S.alloc_planes(planes, N, N, torch.bfloat16, dev)
    wd3 = dict(ln_in_w=ln_in[0], ln_in_b=ln_in[1], w_left=w_gate, w_left_gate=w_gate, w_right=w_gate,
               w_right_gate=w_gate, ln_out_w=t(w.ln_out_weight), ln_out_b=t(w.ln_out_bias), w_gate=w_gate, w_out=w_out)
    wd1 = []
    for direction in (0, 1):
        rows = slice(direction * h, (direction + 1) * h)
        wd1.append(dict(ln_in_w=ln_in[0], ln_in_b=ln_in[1], w_left=wl[rows], w_left_gate=wlg[rows], w_right=wr[rows],
                        w_right_gate=wrg[rows], ln_out_w=ln_in[0], ln_out_b=ln_in[1], w_gate=w_gate, w_out=w_gate))
    views = []
    for direction in (0, 1):
        first = direction * h * a.plane_stride
        views.append(tuple(S.PlaneSpec(sp.buf[first:], h, N, N, sp.pitch, sp.plane_stride) for sp in (a, b)))

    def step(ev=None):
        mark = (lambda: (ev.append(torch.cuda.Event(enable_timing=True)), ev[-1].record())) if ev is not None else (lambda: None)
        mark()
        for direction in (0, 1):
            S.tm1(z, m, wd1[direction], views[direction][0], views[direction][1], outgoing=(direction == 0))
        mark()
        S.contract(a, b, tri)
        mark()
        y = S.tm2(z, tri, wd3, residual=z)
        mark()
        return y

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(0)
    all_ev = []
    for _ in range(args.steps):
        ev = []
        step(ev)
        all_ev.append(ev)
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    if read_status(dev)[0] != 0:
        raise SystemExit(f"bench.py: device status {read_status(dev)}: timing is invalid")
    ms = all_ev[0][0].elapsed_time(all_ev[-1][-1]) / args.steps
    stage_ms = [sum(e[i].elapsed_time(e[i + 1]) for e in all_ev) / args.steps for i in range(3)]
    M = B * N * N
    flops = 22.0 * M * d * d + 4.0 * B * N ** 3 * d      # 4 [2h,d] + [d,d] + [d,2h] projections; 2h planes contracted
    S_bytes = M * d * 2
    peaks = measured_peaks()
    # algorithmic bytes: stage 1 reads z twice and writes 4 S; contraction reads 4 S, writes 2 S; stage 3 reads 3 S, writes S
    alg = {"tm1 x2": 6 * S_bytes, "contract": None, "tm2 (wide)": 4 * S_bytes}
    stages = {}
    for name, v in zip(alg, stage_ms):
        if alg[name] is None:
            ach = 4.0 * B * N ** 3 * d / (v * 1e-3) / 1e12
            stages[name] = {"ms": v, "bound": "tensor", "achieved": ach, "unit": "TFLOP/s",
                            "peak": peaks["bf16_tflops_sustained"], "frac": ach / peaks["bf16_tflops_sustained"]}
        else:
            ach = alg[name] / (v * 1e-3) / 1e9
            stages[name] = {"ms": v, "bound": "hbm", "achieved": ach, "unit": "GB/s", "peak": peaks["hbm_gbs"],
                            "frac": ach / peaks["hbm_gbs"]}
    dom = max(stages, key=lambda k: stages[k]["ms"])
    line = {
        "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "calls_per_s": 1e3 / ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded randn pair tensor and weights, all-ones LayerNorm gamma)",
        "frac_of_bf16_peak": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "config": dict(workload_config(args.workload, B, N, d, "bidirectional (outgoing + incoming halves), residual added",
                                       mask_kind), c_hidden=2 * h),
        "parallelism": "single GPU",
        "gpu_launches": 4 * args.steps,
        "roofline": dict(stages[dom], kernel=dom, peak_source=peaks["source"], traffic=None),
        "stages": stages, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="n768_outgoing", choices=sorted(WORKLOADS) + sorted(PAIR_WORKLOADS) + sorted(BIDIR_WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard-mode", default="auto", choices=["auto", "rows", "channels", "peer"],
                    help="exchange pattern of the *_pair_sharded workloads")
    ap.add_argument("--no-check", action="store_true",
                    help="*_pair_sharded: skip the comparison with the unsharded result")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        run_reference(args)
    else:
        args.steps = 50 if args.steps is None else args.steps
        args.warmup = 5 if args.warmup is None else args.warmup
        if args.workload in PAIR_WORKLOADS:
            run_sharded_pair(args)
        elif args.workload in BIDIR_WORKLOADS:
            run_bidirectional(args)
        else:
            run_b200(args)


if __name__ == "__main__":
    main()
