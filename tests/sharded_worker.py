"""One rank of the multi-GPU sharding test (launched by torch.distributed.run).

Every rank computes its slab of the block with the NCCL exchange and compares it with the
unsharded result computed on its own GPU and with the CPU oracle."""

import argparse
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import trimul_oracle as O  # noqa: E402
from tests._util import forward_kwargs, weights_dict  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--N", type=int, default=512)
    ap.add_argument("--direction", default="outgoing")
    ap.add_argument("--mode", default="rows")
    args = ap.parse_args()
    from miniworld_engine_b200 import read_status, trimul_forward
    from miniworld_engine_b200.sharded import trimul_forward_sharded
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    outgoing = args.direction == "outgoing"
    N, R = args.N, args.N // world
    w = O.make_weights(128, 0, affine="random")
    z = O.make_input(1, N, 128, 1).bfloat16()
    m = O.make_token_mask(1, N, "rand5")
    wd = weights_dict(w, torch.bfloat16, dev)
    slab = z[:, rank * R:(rank + 1) * R].contiguous().to(dev)
    if args.mode == "peer":
        from miniworld_engine_b200.sharded import PeerShardContext
        ctx = PeerShardContext(1, N, 128, torch.bfloat16, dev)
        out = ctx.forward(slab, m.to(dev), wd, outgoing=outgoing)
        out = ctx.forward(slab, m.to(dev), wd, outgoing=outgoing).cpu()     # buffers are reused between calls
    else:
        out = trimul_forward_sharded(slab, m.to(dev), wd, outgoing=outgoing, N=N, mode=args.mode).cpu()
    whole = trimul_forward(z.to(dev), m.to(dev), outgoing=outgoing, **forward_kwargs(w, torch.bfloat16, dev)).cpu()
    assert read_status(dev)[0] == 0
    ref = O.trimul_forward(z, m, w.to(torch.bfloat16), outgoing)[:, rank * R:(rank + 1) * R]
    e_whole = O.rel_rms(out.float(), whole[:, rank * R:(rank + 1) * R].float())
    e_ref = O.rel_rms(out.float(), ref.float())
    ok = torch.tensor([int(e_whole <= 4e-3 and e_ref <= 1e-2)], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    print(f"rank {rank}: vs unsharded {e_whole:.3e}, vs oracle {e_ref:.3e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if int(ok.item()) != 1:
        sys.exit(1)
    if rank == 0:
        print("SHARDED_OK", flush=True)


if __name__ == "__main__":
    main()
