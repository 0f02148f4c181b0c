"""One MoE expert block (dispatch -> fc1 + SwiGLU x weight -> fc2 -> combine, forward and backward) with the token
exchange inside the grouped GEMMs, timed with CUDA events on every rank (max over ranks), next to the same block on the
NCCL all-to-all dispatcher.  With one process the rank pushes to itself through the same kernels, which is the form a
single-kernel `ncu` capture needs:

    python -m torchturbo_b200.benchmarks.ep_fused_bench [--tokens 4096] [--experts 16] [--iters 20]
    torchrun --nproc-per-node N -m torchturbo_b200.benchmarks.ep_fused_bench --experts 128

Shapes default to the Qwen3-30B-A3B layer (hidden 2048, expert FFN 768, top-8); `--experts` is the global expert
count (16 with one process = the per-rank load of an 8-GPU run).  Inputs (x, weights, saved activations) are tens to
hundreds of MB per rank, i.e. larger than L2 only for `--tokens` >= 16384: the numbers are kernel-level, use them to
compare the two dispatchers, not as DRAM roofline points."""
from __future__ import annotations

import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=768)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--forward-only", action="store_true")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29561")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120),
                            device_id=torch.device("cuda", local))
    from .. import kernels
    from ..comm.ep_p2p import _WORKSPACES, P2PTokenDispatcher
    from ..models.modules.moe import MoELayerConfig
    from ..models.modules.moe.moe import MoEAlltoAllTokenDispatcher
    from ..ops import ops

    T, H, F, E, k = args.tokens, args.hidden, args.ffn, args.experts, args.topk
    El = E // world
    cfg = MoELayerConfig(hidden_size=H, moe_ffn_hidden_size=F, num_moe_experts=E, moe_router_topk=k, params_dtype=torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    x = (torch.randn(T, H, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
    w1 = (torch.randn(El, H, 2 * F, device="cuda", generator=g) * 0.02).bfloat16().requires_grad_(True)
    w2 = (torch.randn(El, F, H, device="cuda", generator=g) * 0.02).bfloat16().requires_grad_(True)
    prob, idx = torch.softmax(torch.randn(T, E, device="cuda", generator=g), -1).topk(k, dim=-1)
    prob = (prob / prob.sum(-1, keepdim=True)).float().requires_grad_(True)
    gout = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    fused = P2PTokenDispatcher(cfg, dist.group.WORLD, El)
    nccl = MoEAlltoAllTokenDispatcher(cfg, dist.group.WORLD, El) if world > 1 else None

    def run_fused():
        y = fused.fused_experts(x, idx, prob, w1, w2)
        if not args.forward_only:
            y.backward(gout)

    def run_nccl():
        perm, tpe, state = nccl.dispatch(x, idx, prob)
        y = nccl.combine(ops.moe_experts(perm, w1, w2, tpe), state)
        if not args.forward_only:
            y.backward(gout)

    def timed(fn) -> float:
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {"world": world, "tokens_per_rank": T, "hidden": H, "ffn": F, "experts": E, "topk": k,
           "passes": "forward" if args.forward_only else "forward+backward", "fused_ms": timed(run_fused)}
    if nccl is not None:
        out["nccl_ms"] = timed(run_nccl)
    flops = 2.0 * T * k * H * 3 * F * (1 if args.forward_only else 3)          # per rank, balanced routing
    out["fused_tflops_per_gpu"] = flops / (out["fused_ms"] * 1e-3) / 1e12
    for ws in _WORKSPACES.values():
        ws.check()
    out["status"] = [kernels.status(), kernels.comm_status()]
    if rank == 0:
        print(json.dumps(out))
    _WORKSPACES.clear()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
