"""Bandwidth of the peer-memory FSDP collectives against NCCL on the same buffers.

    torchrun --nproc-per-node N -m torchturbo_b200.benchmarks.peer_collective_bench [--mb 64 256 1024] [--grids 16 48 96] [--ep]

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
    ap.add_argument("--ep", action="store_true", help="also time the expert-parallel row scatter / gather")
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
    if args.ep:
        _bench_ep(args, g, rank, world, dev)
    dist.barrier()
    dist.destroy_process_group()


def _bench_ep(args, g, rank, world, dev) -> None:
    """Expert-parallel row exchange at the 30B-A3B layer shape: 4096 tokens x top-8 of 128 experts, hidden 2048.
    Scatter pushes every routed row into its owner's buffer, gather pulls the k expert outputs of every token back and
    sums them; the bytes that cross NVLink are the rows whose expert lives on another rank."""
    from .. import kernels as K
    from ..comm import ep_p2p

    T, H, E, k = 4096, 2048, 128, 8
    torch.manual_seed(7 + rank)
    x = torch.randn(T, H, device=dev).bfloat16()
    idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32)
    prob = torch.rand(T, k, device=dev)
    ws = ep_p2p.get_workspace(g, H, E, T, k, 2.0)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    counts.scatter_add_(0, idx.reshape(-1).long(), torch.ones(T * k, dtype=torch.int32, device=dev))
    seg_start, recv_counts, tile_group, dest_base = ws.exchange(counts)
    expert = idx.reshape(-1).contiguous()
    dest_row = K.perm_rank(expert, E, dest_base)
    pflat = prob.reshape(-1).contiguous()
    remote = int(((expert // (E // world)) != rank).sum().item())
    nbytes = remote * H * 2

    def scatter():
        ws.scatter_rows(x, expert, dest_row, pflat, k)

    def gather():
        ws.publish_and_wait_ready()
        ws.gather_rows(expert, dest_row, T, k)

    t_s, t_g = _time(scatter, args.iters, g), _time(gather, args.iters, g)
    torch.cuda.synchronize()
    ws.check()
    if rank == 0:
        print(f"EP rows (T={T}, k={k}, E={E}, H={H}, {world} ranks): {remote} of {T * k} rows remote = {nbytes / 1e6:.1f} MB; "
              f"scatter + landed-wait {t_s:.3f} ms {nbytes / t_s / 1e6:.1f} GB/s | ready-wait + gather-sum {t_g:.3f} ms "
              f"{nbytes / t_g / 1e6:.1f} GB/s", flush=True)


if __name__ == "__main__":
    main()
