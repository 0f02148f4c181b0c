"""Expert-parallel exchange fused into the grouped GEMMs (push prologue / scatter epilogue of csrc/gemm.cu).

Every case compares one MoE expert block (dispatch -> fc1 -> SwiGLU x weight -> fc2 -> combine, forward and backward)
with a plain fp32 torch formulation over the full expert set; the multi-GPU cases also run the NCCL all-to-all
dispatcher of the same package on the same inputs.  World 1 runs on a single GPU (the rank pushes to itself), worlds 2
and 4 start one process per GPU with NVLS off; one rank sleeps on the host between layers so that peers run ahead as
far as the flags allow (buffer reuse under skew)."""
import os
import tempfile
import time
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu

H, F, E, TOPK = 256, 128, 16, 4


def _oracle(x, idx, prob, W1, W2, residual=None):
    """fp32: out[t] = sum_j prob[t, j] * (silu(x W1g[e]) * (x W1u[e])) W2[e],  e = idx[t, j]."""
    xf = x.float()
    out = torch.zeros_like(xf)
    for j in range(idx.shape[1]):
        e = idx[:, j].long()
        h = torch.bmm(xf[:, None, :], W1.float()[e]).squeeze(1)
        a = torch.nn.functional.silu(h[:, :F]) * h[:, F:] * prob[:, j:j + 1].float()
        out = out + torch.bmm(a[:, None, :], W2.float()[e]).squeeze(1)
    return out if residual is None else out + residual.float()


def _close(u, v, what, tol=3e-2):
    err = (u.float() - v.float()).abs().max().item()
    ref = v.float().abs().max().item()
    assert err <= tol * max(ref, 1e-3), f"{what}: err {err} ref {ref}"


def _worker(rank, world, init_file, err_dir, skew):
    try:
        import datetime

        import torch.distributed as dist

        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["LOCAL_RANK"] = str(rank)
        os.environ["TORCHTURBO_P2P_WAIT_MS"] = "20000"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
        from torchturbo_b200 import kernels
        from torchturbo_b200.comm.ep_p2p import _WORKSPACES, P2PTokenDispatcher
        from torchturbo_b200.models.modules.moe import MoELayerConfig
        from torchturbo_b200.models.modules.moe.moe import MoEAlltoAllTokenDispatcher
        from torchturbo_b200.ops import ops

        os.environ["TORCHTURBO_EP_MAX_TOKENS"] = "2048"
        cfg = MoELayerConfig(hidden_size=H, moe_ffn_hidden_size=F, num_moe_experts=E, moe_router_topk=TOPK,
                             params_dtype=torch.bfloat16)
        El = E // world
        g = torch.Generator(device="cuda").manual_seed(7)
        W1 = (torch.randn(E, H, 2 * F, device="cuda", generator=g) * 0.05).bfloat16()
        W2 = (torch.randn(E, F, H, device="cuda", generator=g) * 0.05).bfloat16()
        sl = slice(rank * El, (rank + 1) * El)
        disp = P2PTokenDispatcher(cfg, dist.group.WORLD, El)
        nccl = MoEAlltoAllTokenDispatcher(cfg, dist.group.WORLD, El) if world > 1 else None
        steps = [(300 + 57 * rank, False), (1900 - 230 * rank, True), (64 + rank, False), (1000, True)]
        for step, (T, with_res) in enumerate(steps):
            torch.manual_seed(100 + 10 * step + rank)
            x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
            res = (torch.randn(T, H, device="cuda") * 0.5).bfloat16() if with_res else None
            logits = torch.randn(T, E, device="cuda")
            if step == 2:          # adversarial routing: every token of every rank goes to the experts of rank 0
                logits[:, El:] -= 100.0
            prob, idx = torch.softmax(logits, -1).topk(TOPK, dim=-1)
            prob = (prob / prob.sum(-1, keepdim=True)).float()
            gout = torch.randn(T, H, device="cuda").bfloat16()
            if skew and rank == world - 1:
                torch.cuda.synchronize()
                time.sleep(0.3)     # the other ranks run ahead until a flag of this rank stops them
            # ---- fused kernels
            xa, pa = x.clone().requires_grad_(True), prob.clone().requires_grad_(True)
            w1a, w2a = W1[sl].clone().requires_grad_(True), W2[sl].clone().requires_grad_(True)
            ya = disp.fused_experts(xa, idx, pa, w1a, w2a, residual=res)
            ya.backward(gout)
            # ---- fp32 oracle over the full expert set (weight gradients summed over the ranks' tokens)
            xo, po = x.float().requires_grad_(True), prob.clone().requires_grad_(True)
            W1o, W2o = W1.float().requires_grad_(True), W2.float().requires_grad_(True)
            yo = _oracle(xo, idx, po, W1o, W2o, res)
            yo.backward(gout.float())
            if world > 1:
                dist.all_reduce(W1o.grad)
                dist.all_reduce(W2o.grad)
            torch.cuda.synchronize()
            for ws in _WORKSPACES.values():
                ws.check()
            tag = f"(world {world}, rank {rank}, step {step})"
            _close(ya, yo, "output vs oracle " + tag)
            _close(xa.grad, xo.grad, "dx vs oracle " + tag)
            _close(pa.grad, po.grad, "dprob vs oracle " + tag, tol=5e-2)
            _close(w1a.grad, W1o.grad[sl], "dw1 vs oracle " + tag)
            _close(w2a.grad, W2o.grad[sl], "dw2 vs oracle " + tag)
            # ---- NCCL all-to-all dispatcher of the same package
            if nccl is not None:
                xb, pb = x.clone().requires_grad_(True), prob.clone().requires_grad_(True)
                w1b, w2b = W1[sl].clone().requires_grad_(True), W2[sl].clone().requires_grad_(True)
                perm, tpe, state = nccl.dispatch(xb, idx, pb)
                yb = nccl.combine(ops.moe_experts(perm, w1b, w2b, tpe), state)
                if res is not None:
                    yb = yb + res
                yb.backward(gout)
                _close(ya, yb, "output vs nccl " + tag)
                _close(xa.grad, xb.grad, "dx vs nccl " + tag)
                _close(w1a.grad, w1b.grad, "dw1 vs nccl " + tag)
        assert kernels.comm_status() == (0, 0) and kernels.status() == (0, 0)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


def _run(world, skew):
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker, args=(world, os.path.join(d, "rdzv"), d, skew), nprocs=world, join=True,
                               start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise


def _worker_overflow(rank, world, init_file, err_dir, _skew):
    """Adversarial routing: every token of every rank picks experts of rank 0, with a receive capacity of 1.0 x the
    balanced share.  The layer's exchange is dropped as a whole (no row is written anywhere), the workspace status
    poisons the gradient norm on the device, the optimizer update is skipped and the step's own finite check raises
    `EPCapacityExceeded` on every rank; with retries allowed the buffers are doubled and the step is repeated."""
    try:
        import datetime

        import torch.distributed as dist

        os.environ.update({"NCCL_NVLS_ENABLE": "0", "LOCAL_RANK": str(rank), "RANK": str(rank), "WORLD_SIZE": str(world),
                           "TORCHTURBO_EP_CAPACITY_FACTOR": "1.0", "TORCHTURBO_P2P_WAIT_MS": "20000"})
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
        from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
        from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
        from torchturbo_b200.engine.optimizers import OptimizerClassPlan
        from torchturbo_b200.loops import train_step
        from torchturbo_b200.models.modules.moe import MoELayer

        eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "bf16", "parallel_plan": {"sp_size": 1, "ep_size": world},
                                                       "activation_checkpointing": {"enabled": False}}))
        mc = dict(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                  num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_experts=16, num_experts_per_tok=4,
                  moe_intermediate_size=256, norm_topk_prob=True)
        model = eng.build_model(None, load_weights=False, init_kwargs={"config": mc})
        opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3))
        ds = SyntheticPackedDataset(8, 1024, mc["vocab_size"], min_doc=128, max_doc=700, seed=0)

        def batch(i):
            b = PackedCollator()([ds[rank * 4 + i]])
            return {k: (v.cuda() if isinstance(v, torch.Tensor) and not k.startswith("cu_seq") else v) for k, v in b.items()}

        loss, _ = train_step(eng, model, opt, [batch(0)])          # balanced routing: fine
        assert torch.isfinite(loss)
        before = [p.detach().clone() for p in model.parameters()]
        for m in model.modules():
            if isinstance(m, MoELayer):
                orig = m.router.forward

                def skewed(x, input_ids=None, runtime=None, _orig=orig, _router=m.router):
                    idx, prob, logits = _orig(x, input_ids, runtime)
                    _router.last_counts = None          # the kernel's histogram belongs to the routing it replaced
                    return torch.arange(idx.shape[1], device=idx.device, dtype=idx.dtype).expand_as(idx).contiguous(), prob, logits

                m.router.forward = skewed
        from torchturbo_b200.comm.ep_p2p import _WORKSPACES, EPCapacityExceeded

        def params():
            return [(p._local_tensor if hasattr(p, "_local_tensor") else p).detach().clone() for p in model.parameters()]

        # (1) no retry allowed: the step raises on every rank, names the overflow, and no weight has changed
        with pytest.raises(EPCapacityExceeded, match="capacity"):
            train_step(eng, model, opt, [batch(1)], ep_overflow_retries=0)
        for p, q in zip(params(), before):
            ql = q._local_tensor if hasattr(q, "_local_tensor") else q
            assert torch.equal(p, ql), "the optimizer stepped on a batch whose rows were not exchanged"
        # (2) default: buffers are doubled (capacity 1.0 -> 2.0 covers "everything to one of two ranks") and the step is
        #     repeated; it must now train, on a clean status
        eng.recover_from_ep_overflow(opt)
        cf0 = [ws.capacity_factor for ws in _WORKSPACES.values()]
        os.environ["TORCHTURBO_EP_CAPACITY_FACTOR"] = "1.0"
        for key in list(_WORKSPACES):      # back to the small buffers so that the step itself has to grow them
            ws = _WORKSPACES.pop(key)
            _WORKSPACES[key] = type(ws)(ws.group, ws.H, ws.E, ws.tokens, ws.topk, 1.0)
            del ws
        loss, gnorm = train_step(eng, model, opt, [batch(1)])
        assert torch.isfinite(loss) and torch.isfinite(gnorm)
        assert all(ws.capacity_factor == 2.0 for ws in _WORKSPACES.values()), (cf0, [ws.capacity_factor for ws in _WORKSPACES.values()])
        assert any(not torch.equal(p, (q._local_tensor if hasattr(q, "_local_tensor") else q)) for p, q in zip(params(), before))
        eng.check_health()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_receive_overflow_is_caught_in_the_same_step_then_recovered_by_growing_the_buffers():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker_overflow, args=(2, os.path.join(d, "rdzv"), d, False), nprocs=2, join=True,
                               start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise


def test_fused_exchange_single_rank_matches_oracle():
    """World 1: the push warps write into this GPU's own receive buffer and the scatter epilogue into its own return
    buffer, so the whole fused path (flags included) runs on one GPU."""
    _run(1, False)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_exchange_two_ranks_matches_oracle_and_nccl():
    _run(2, True)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_fused_exchange_four_ranks_matches_oracle_and_nccl():
    _run(4, True)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_fused_exchange_eight_ranks_matches_oracle_and_nccl():
    _run(8, True)
