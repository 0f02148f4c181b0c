"""Headline benchmark: SFT tokens/s of a Qwen3-30B-A3B-shaped MoE (FSDP2 + EP) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...      # same metric through the unmodified reference (baseline/_ref)

Prints ONE JSON line on rank 0.  `value` is the device-timed aggregate tokens/s over K steps (CUDA events, barrier
and synchronize on both sides, max over ranks); `e2e` repeats the measurement through the public engine API with the
per-step host-to-device copy of the batch from pinned memory and the device-to-host read of the loss inside the timed
region.  Synthetic data (seeded random token ids, documents of 256..4096 tokens packed to 4096 per rank), random-init
weights, bf16 compute with fp32 master weights and optimizer state, AdamW, global-norm clipping, aux loss 1e-3.
After the W warm-up steps both arms keep warming up (each extra step timed on its own) until two consecutive steps
differ by less than 3 % or 12 extra steps have run; `warmup_used` reports the total.

Depth: the named model has 48 layers; its fp32 master + AdamW state (16 bytes per parameter) only fits when the
experts are spread over 4 or more GPUs, so `layers = min(48, 12 * N)`; the depth used is reported in `config`.
Because that changes the work per GPU between N = 1, 2 and 4, the line also carries `fixed_depth`: the same
measurement at 12 layers for every N, which is the series to read scaling from.

With 8 GPUs the line also carries `secondary`: the other named 8-GPU configurations (Qwen3-14B shape, Ulysses sp = 8,
one 65536-token row per group; Qwen3-8B shape, FSDP over 8, 8192-token rows), each measured the same way in fresh
processes that rank 0 starts after the headline run has released the GPUs (`--extras none|fixed|all` overrides).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "SFT tokens/s, Qwen3-30B-A3B FSDP2+EP, aggregate over N B200 (device-timed, max over ranks)"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=0, help="0 = min(48, 12 * gpus)")
    p.add_argument("--seq-len", type=int, default=4096)
    p.add_argument("--model", default="qwen3_moe_30b_a3b", choices=["qwen3_moe_30b_a3b", "qwen3_8b", "qwen3_14b", "qwen3_vl_8b", "tiny_moe", "tiny_dense"])
    p.add_argument("--sp", type=int, default=1, help="Ulysses sequence-parallel size (a sequence of --seq-len tokens per SP group)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--fsdp-transport", default="auto", choices=["auto", "nccl", "p2p"],
                   help="all-gather / reduce-scatter of the FSDP units: peer-memory kernels (auto / p2p) or NCCL")
    p.add_argument("--fsdp-unit-mb", type=int, default=-1, help="merge decoder layers into FSDP units of at least "
                   "this many MiB of bf16 parameters (-1: engine default, 0: one unit per layer)")
    p.add_argument("--ep-transport", default="auto", choices=["auto", "nccl", "p2p"],
                   help="expert-parallel token exchange: NVLink peer-memory kernels (p2p) or NCCL all-to-all")
    p.add_argument("--extras", default="auto", choices=["auto", "none", "fixed", "all"],
                   help="records attached to the headline line: fixed-depth (12-layer) run, secondary named configs "
                        "(auto: fixed-depth from 2 GPUs on, secondaries at 8 GPUs)")
    p.add_argument("--extras-budget-s", type=float, default=600.0, help="wall-clock budget of the whole call; an extra "
                   "record is only started while enough of it is left")
    p.add_argument("--child", action="store_true", help=argparse.SUPPRESS)   # a sub-measurement started by rank 0
    return p.parse_args()


def model_config(name: str, layers: int) -> dict:
    if name == "qwen3_moe_30b_a3b":
        return dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                    num_hidden_layers=layers, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                    num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
                    rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, router_aux_loss_coef=1e-3)
    if name == "qwen3_14b":
        return dict(model_type="qwen3", vocab_size=151936, hidden_size=5120, intermediate_size=17408,
                    num_hidden_layers=layers, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                    rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)
    if name == "qwen3_8b":
        return dict(model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                    num_hidden_layers=layers, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                    rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)
    if name == "qwen3_vl_8b":
        # 27-layer ViT (width 1152, 16 heads, MLP 4304, patch 14, 2x2 merge) in front of the Qwen3-8B decoder
        text = model_config("qwen3_8b", layers)
        text.pop("model_type")
        return dict(model_type="qwen3_vl", text_config=text, vision_config=dict(depth=27, hidden_size=1152, num_heads=16,
                    intermediate_size=4304, patch_size=14, temporal_patch_size=2, spatial_merge_size=2), vocab_size=151936)
    if name == "tiny_dense":
        return dict(model_type="qwen3", vocab_size=32000, hidden_size=512, intermediate_size=1024, num_hidden_layers=layers,
                    num_attention_heads=8, num_key_value_heads=2, head_dim=128, rope_theta=1e6, rms_norm_eps=1e-6,
                    tie_word_embeddings=False)
    return dict(model_type="qwen3_moe", vocab_size=32000, hidden_size=512, intermediate_size=1024,
                num_hidden_layers=layers, num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_experts=16,
                num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True)


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, f"/tmp/ttb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx = float(parts[1])
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from torchturbo_b200 import kernels
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    named_layers = {"qwen3_moe_30b_a3b": 48, "qwen3_8b": 36, "qwen3_14b": 40, "qwen3_vl_8b": 36}.get(args.model, 4)
    layers = args.layers or min(named_layers, 12 * world)
    is_vlm = args.model == "qwen3_vl_8b"
    is_moe = args.model not in ("qwen3_8b", "qwen3_14b", "tiny_dense", "qwen3_vl_8b")
    sp = max(args.sp, 1)
    cfg = EngineConfig.from_dict({
        "mixed_precision": "bf16",
        "parallel_plan": {"sp_size": sp, "ep_size": world if is_moe else 1},
        "moe": {"aux_loss_coeff": 1e-3},
        "activation_checkpointing": {"enabled": not is_moe},
        **({"parallel_plan": {"sp_size": sp, "ep_size": 1, "plan": {"model.visual": {"vision_balance": {"mode": "patch_sq"}}}}}
           if is_vlm else {}),
        "backend_config": dict({"transport": args.fsdp_transport},
                               **({"unit_min_bytes": args.fsdp_unit_mb << 20} if args.fsdp_unit_mb >= 0 else {})),
    })
    engine = TorchTurboEngine(cfg)
    mc = model_config(args.model, layers)
    if is_moe:
        mc["moe_token_dispatcher_transport"] = args.ep_transport
    model = engine.build_model(None, load_weights=False, init_kwargs={"config": mc, "seed": 0})
    optim = engine.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-5, weight_decay=0.01,
                                                               betas=(0.9, 0.95)))
    n_batches = max(args.warmup, 1) + 2 * args.steps
    if is_vlm:
        # one sample per rank: `seq_len` text tokens plus 0..8 images of 224..1344 pixels a side (placeholders inserted);
        # the images of all ranks are pooled and spread by squared patch count before the vision tower runs
        from torchturbo_b200.data import SyntheticVLMDataset

        ds = SyntheticVLMDataset(n_batches * world, args.seq_len, mc["vocab_size"], image_token_id=151655,
                                 vision_start_token_id=151652, seed=1234)
        host = [{k: (v.pin_memory() if isinstance(v, torch.Tensor) and not k.startswith("cu_seq") else v)
                 for k, v in ds[(rank // sp) * n_batches + i].items()} for i in range(n_batches)]
    else:
        ds = SyntheticPackedDataset(n_batches * world, args.seq_len, mc["vocab_size"], min_doc=256, max_doc=args.seq_len,
                                    seed=1234)
        coll = PackedCollator(pin=True)
        host = [coll([ds[(rank // sp) * n_batches + i]]) for i in range(n_batches)]   # an SP group shares its row

    def tokens_in(batches) -> float:
        """Tokens of the given steps summed over the data-parallel groups (rows differ in length with images)."""
        n = torch.tensor([float(sum(int(b["input_ids"].numel()) for b in batches))], device=torch.device("cuda", local_rank))
        if world > 1:
            dist.all_reduce(n)
        return float(n.item()) / sp
    dev = torch.device("cuda", local_rank)

    def to_device(b):
        return {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) and not k.startswith("cu_seq") else v)
                for k, v in b.items()}

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    model.train()
    # ---- warm-up: W steps, then until two consecutive steps agree within 3 % (at most EXTRA_WARMUP more)
    # Warm-up steps read their loss / norm on the host (`check_finite`): random-init routers send very uneven loads, and
    # a step whose expert exchange overflows its receive buffers is repeated with larger ones here, so that the timed
    # steps (which read nothing) run with buffers that fit.  `peer_status` below proves that no timed step overflowed.
    for i in range(args.warmup):
        train_step(engine, model, optim, [to_device(host[i])], check_finite=True)
    warmup_used = args.warmup + stabilise(lambda j: train_step(engine, model, optim, [to_device(host[j % args.warmup])],
                                                               check_finite=True), sync, world, dev,
                                          4 if args.child else EXTRA_WARMUP)
    # ---- device-timed region: inputs staged on the device beforehand
    staged = [to_device(host[args.warmup + i]) for i in range(args.steps)]
    sampler = ClockSampler(local_rank)
    sync()
    sampler.start()
    launches0 = kernels.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for b in staged:
        last, _ = train_step(engine, model, optim, [b], check_finite=False)
    e1.record()
    sync()
    launches = kernels.launch_count() - launches0
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev = float(t.item())
    tokens_per_step = args.seq_len * (world // sp)
    timed_tokens = tokens_in(host[args.warmup:args.warmup + args.steps]) if is_vlm else tokens_per_step * args.steps
    value = timed_tokens / (ms_dev / 1e3)
    # ---- end-to-end region: public API, H2D of every batch from pinned memory, D2H of every loss
    e2e = None
    if not args.no_e2e:
        h2d = sum(v.numel() * v.element_size() for k, v in host[0].items()
                  if isinstance(v, torch.Tensor) and not k.startswith("cu_seq"))
        losses = []
        sync()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            b = to_device(host[args.warmup + args.steps + i])
            loss, _ = train_step(engine, model, optim, [b], check_finite=False)
            losses.append(float(loss.cpu()))        # device -> host read of the step's result
        f1.record()
        sync()
        t2 = torch.tensor([f0.elapsed_time(f1)], device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e_tokens = (tokens_in(host[args.warmup + args.steps:args.warmup + 2 * args.steps]) if is_vlm
                      else tokens_per_step * args.steps)
        e2e = {"value": e2e_tokens / (float(t2.item()) / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4, "ms_per_step": float(t2.item()) / args.steps,
               "final_loss": losses[-1]}
    st = kernels.status()
    # status words of every peer-memory workspace (expert-parallel, Ulysses, FSDP arenas): a timeout or a receive
    # overflow anywhere in the run would make the number above meaningless
    try:
        engine.check_health()
        peer_status = "ok"
    except Exception as e:  # noqa: BLE001
        peer_status = f"{type(e).__name__}: {e}"[:200]
    try:
        from torchturbo_b200.comm import ep_p2p

        ep_capacity = max([ws.capacity_factor for ws in ep_p2p._WORKSPACES.values()], default=None)
    except Exception:  # noqa: BLE001
        ep_capacity = None
    disp = [type(m.token_dispatcher).__name__ for m in model.modules() if hasattr(m, "token_dispatcher")]
    ep_transport = (disp[0] if disp else "none") if world > 1 else "local"
    out = {
        "metric": METRIC if args.model == "qwen3_moe_30b_a3b" else METRIC.replace("Qwen3-30B-A3B FSDP2+EP", args.model), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random token ids, random-init weights)", "impl": "ours",
        "config": {"model": "Qwen3-30B-A3B" if args.model == "qwen3_moe_30b_a3b" else args.model, "layers": layers,
                   "layers_named": named_layers, "global_batch": world // sp, "seq_len": args.seq_len,
                   "parallelism": f"fsdp2 dp{world // sp} + ep{world if is_moe else 1}" + (f" + ulysses sp{sp}" if sp > 1 else ""),
                   "sp_transport": os.environ.get("TORCHTURBO_ULYSSES_TRANSPORT", "auto") if sp > 1 else "none", "optimizer": "AdamW fp32 master",
                   "ep_transport": ep_transport, "ep_receive_capacity_x_balanced": ep_capacity,
                   "fsdp_transport": "p2p" if getattr(engine.backend, "peer_arenas", None) else ("nccl" if world > 1 else "local"),
                   "fsdp_units": len(engine.backend.fsdp_units),
                   "reshard_after_forward": engine.backend.fsdp_config.reshard_after_forward, "depth_rule": f"layers = min({named_layers}, 12 * n_gpus): the deepest stack whose "
                   "weights + fp32 AdamW state fit 180 GB per GPU without activation checkpointing; the named "
                   "depth from 4 GPUs on", "tokens_per_s_scaled_to_named_layers": value * layers / float(named_layers),
                   "l2": "per-step working set (weights, optimizer state, activations: tens of GB) is far larger than the 126 MB L2"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "loss": float(last),
        "kernel_status": list(st), "peer_status": peer_status, "warmup_used": warmup_used,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
    }
    if peer_status != "ok":
        out["invalid"] = "a peer-memory exchange failed inside the measured steps: " + peer_status
    # every rank lets go of its peer-mapped buffers before any of them leaves (rank 0 carries on with other work)
    del optim
    engine.close(model)
    del model
    if dist.is_initialized():
        dist.destroy_process_group()
    return out if rank == 0 else {}


EXTRA_WARMUP = 12


def stabilise(step_fn, sync, world, dev, limit: int = EXTRA_WARMUP) -> int:
    """Extra warm-up: runs single steps, each timed on the device (max over ranks), until two consecutive ones differ
    by less than 3 % or `limit` steps have run.  Returns how many ran."""
    import torch
    import torch.distributed as dist

    prev, used = None, 0
    while used < limit:
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step_fn(used)
        b.record()
        sync()
        t = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        cur = float(t.item())
        used += 1
        if prev is not None and abs(cur - prev) <= 0.03 * max(cur, prev):
            break
        prev = cur
    return used


_LAUNCHER_ENV = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_NAME",
                 "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RESTART_COUNT",
                 "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_RUN_ID", "TORCHELASTIC_USE_AGENT_STORE",
                 "TORCHELASTIC_ERROR_FILE", "TORCH_NCCL_ASYNC_ERROR_HANDLING")


def run_child(args, world: int, extra: list[str], timeout_s: float) -> dict:
    """One more measurement in fresh processes (same arm, same launch form as this call); returns its JSON record."""
    env = {k: v for k, v in os.environ.items() if k not in _LAUNCHER_ENV}
    me = os.path.abspath(__file__)
    base = [sys.executable]
    if world > 1:
        port = 29700 + (os.getpid() % 200)
        base += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                 "--master-port", str(port)]
    cmd = base + [me, "--child", "--extras", "none", "--impl", args.impl, "--gpus", str(world), "--steps", str(min(args.steps, 4)),
                  "--warmup", str(max(args.warmup, 3))] + extra
    try:
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"error": f"no result within {timeout_s:.0f} s"}
    for line in reversed(res.stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    tail = (res.stderr or "").strip().splitlines()[-1:] or [""]
    return {"error": f"exit {res.returncode}: {tail[0][:200]}"}


def slim(rec: dict) -> dict:
    """The fields of a sub-measurement that the headline line carries."""
    keep = ("impl", "unavailable", "error", "value", "unit", "ms_per_step", "n_gpus", "steps", "warmup", "warmup_used", "e2e",
            "clocks", "gpu_launches", "loss", "peak_mem_gb", "peer_status", "kernel_status", "dtype")
    out = {k: rec[k] for k in keep if k in rec}
    if "config" in rec:
        out["config"] = {k: rec["config"][k] for k in ("model", "layers", "layers_named", "global_batch", "seq_len", "parallelism",
                                                        "activation_checkpointing", "sp_transport", "ep_transport", "fsdp_transport")
                         if k in rec["config"]}
    return out


def extras(args, out: dict, world: int, t_start: float) -> None:
    """Attach `fixed_depth` and `secondary` to the headline record (rank 0, after the GPUs were released)."""
    mode = args.extras
    if mode == "none" or args.model != "qwen3_moe_30b_a3b" or args.sp != 1 or args.layers:
        return
    left = lambda: args.extras_budget_s - (time.time() - t_start)   # noqa: E731
    # ---- the same model at 12 layers for every N: the like-for-like scaling series
    if out.get("config", {}).get("layers") == 12:
        out["fixed_depth"] = slim(out)
    elif mode in ("auto", "fixed", "all") and left() > 150:
        out["fixed_depth"] = slim(run_child(args, world, ["--layers", "12"], min(300.0, left() - 30)))
    # ---- the other named configurations of the 8-GPU box
    if mode == "all" or (mode == "auto" and world >= 8):
        out["secondary"] = []
        for extra in (["--model", "qwen3_14b", "--sp", str(world), "--seq-len", "65536", "--layers", "40"],
                      ["--model", "qwen3_8b", "--seq-len", "8192", "--layers", "36"],
                      ["--model", "qwen3_vl_8b", "--sp", "2", "--seq-len", "4096", "--layers", "36"]):
            if left() < 200:
                out["secondary"].append({"config": {"model": extra[1]}, "error": "skipped: wall-clock budget of the call used up"})
                continue
            out["secondary"].append(slim(run_child(args, world, extra, min(420.0, left() - 30))))


def main():
    t_start = time.time()
    args = parse()
    # stdout carries the one JSON result line: the package's log lines go to stderr
    import logging

    from torchturbo_b200.logging import logging_configure

    logging_configure()
    for h in logging.getLogger("torchturbo_b200").handlers:
        if hasattr(h, "setStream"):
            h.setStream(sys.stderr)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        from baseline.run_reference import run_reference

        out = run_reference(args)
    else:
        out = run_ours(args)
    if out and not args.child and "unavailable" not in out:
        # the other ranks have returned and exit now; this rank drops what it holds on its GPU, then starts the
        # additional measurements as fresh process groups
        try:
            import gc

            import torch

            if args.impl != "reference":
                from torchturbo_b200.comm import ep_p2p, fsdp_p2p, rows_p2p, ulysses_p2p

                for table in (ep_p2p._WORKSPACES, fsdp_p2p._ARENAS, ulysses_p2p._WORKSPACES, rows_p2p._WS):
                    table.clear()
            gc.collect()
            torch.cuda.empty_cache()
        except Exception:  # noqa: BLE001
            pass
        extras(args, out, world, t_start)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
