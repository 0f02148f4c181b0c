"""Bandwidth of the peer-memory FSDP collectives against NCCL on the same buffers.

    torchrun --nproc-per-node N -m torchturbo_b200.benchmarks.peer_collective_bench [--mb 64 256 1024] [--grids 16 48 96]

For every size (MiB of the gathered / scattered buffer per rank) rank 0 prints the time (CUDA events, max over ranks,
mean of `--iters` calls after warm-up) and the bytes this rank moves over NVLink divided by it:
all-gather pulls (W-1)/W of the buffer, reduce-scatter reads (W-1)/W of one piece from the peers.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def _time(fn, iters: int, group) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, nargs="+", default=[64, 256, 1024])
    ap.add_argument("--grids", type=int, nargs="+", default=[16, 48, 96])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ..comm import fsdp_p2p

    g = dist.group.WORLD
    dev = torch.device("cuda", torch.cuda.current_device())
    top = max(args.mb) << 20
    arena = fsdp_p2p.PeerCollectiveArena(g, ag_bytes=top, rs_bytes=top, n_ag=2, n_rs=2)
    ag, rs = fsdp_p2p.PeerAllGather(arena), fsdp_p2p.PeerReduceScatter(arena)
    for mb in args.mb:
        n = (mb << 20) // 2          # bf16 elements of the whole buffer
        piece = n // world
        shard = torch.randn(piece, device=dev).bfloat16()
        ref_out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        t_nccl_ag = _time(lambda: dist.all_gather_into_tensor(ref_out, shard), args.iters, g)
        n32 = (mb << 20) // 4
        grads = torch.randn(n32, device=dev)
        red = torch.empty(n32 // world, device=dev)
        t_nccl_rs = _time(lambda: dist.reduce_scatter_tensor(red, grads, op=dist.ReduceOp.AVG), args.iters, g)
        moved = (mb << 20) * (world - 1) / world
        if rank == 0:
            print(f"{mb:5d} MiB  nccl all-gather {t_nccl_ag:7.3f} ms {moved / t_nccl_ag / 1e6:7.1f} GB/s | "
                  f"nccl reduce-scatter(fp32) {t_nccl_rs:7.3f} ms {moved / world / t_nccl_rs / 1e6 * world:7.1f} GB/s", flush=True)
        for grid in args.grids:
            arena.grid = grid

            def do_ag():
                out = ag.allocate((n,), dtype=torch.bfloat16, device=dev)
                ag(output_tensor=out, input_tensor=out[rank * piece:(rank + 1) * piece], group=g)

            def do_rs():
                inp = rs.allocate((n32,), dtype=torch.float32, device=dev)
                res = rs.allocate((n32 // world,), dtype=torch.float32, device=dev)
                rs(output_tensor=res, input_tensor=inp, group=g, op=dist.ReduceOp.AVG)

            t_ag, t_rs = _time(do_ag, args.iters, g), _time(do_rs, args.iters, g)
            if rank == 0:
                print(f"{mb:5d} MiB  grid {grid:3d}: peer all-gather {t_ag:7.3f} ms {moved / t_ag / 1e6:7.1f} GB/s | "
                      f"peer reduce-scatter(fp32) {t_rs:7.3f} ms {moved / t_rs / 1e6:7.1f} GB/s", flush=True)
    torch.cuda.synchronize()
    arena.check()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
