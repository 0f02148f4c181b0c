"""2-GPU checks of the peer-memory FSDP collectives: the all-gather / reduce-scatter objects against NCCL over many
calls (slot reuse, both dtypes, oversize fallback), and a short training run with the kernels installed into the FSDP
units against the same run on NCCL."""
import os
import tempfile
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu

DENSE = dict(model_type="qwen3", num_hidden_layers=4, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
             head_dim=128, intermediate_size=512, vocab_size=2048, tie_word_embeddings=False)


def _train(transport, steps=4):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    eng = TorchTurboEngine(EngineConfig.from_dict({
        "mixed_precision": "bf16", "parallel_plan": {"sp_size": 1, "ep_size": 1},
        "activation_checkpointing": {"enabled": False},
        "backend_config": {"transport": transport, "unit_min_bytes": 0, "reshard_after_forward": True}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(DENSE), "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3, weight_decay=0.0))
    seen = []
    model.register_forward_pre_hook(lambda m, a, kw: seen.append(kw["cu_seq_lens_q"].device.type), with_kwargs=True)
    ds = SyntheticPackedDataset(2 * steps, 512, DENSE["vocab_size"], num_docs=3, seed=5)
    dp = eng.get_dp_info()
    out = []
    for i in range(steps):
        b = PackedCollator()([ds[i * dp["dp_size"] + dp["dp_rank"]]])
        loss, gn = train_step(eng, model, opt, [b])
        out.append((float(loss), float(gn)))
    # the packed-row boundaries reach the model as host tensors: FSDP's input mover did not copy them to the GPU
    assert seen and set(seen) == {"cpu"}, seen
    return out, eng


def _worker(rank, world, init_file, err_dir):
    try:
        import datetime

        import torch.distributed as dist

        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["LOCAL_RANK"] = str(rank)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
        from torchturbo_b200 import kernels
        from torchturbo_b200.comm import fsdp_p2p

        g = dist.group.WORLD
        dev = torch.device("cuda", rank)
        arena = fsdp_p2p.PeerCollectiveArena(g, ag_bytes=1 << 20, rs_bytes=2 << 20, n_ag=3, n_rs=2)
        ag, rs = fsdp_p2p.PeerAllGather(arena), fsdp_p2p.PeerReduceScatter(arena)
        side = torch.cuda.Stream()
        for it in range(9):                      # more calls than slots: every slot is reused several times
            dt = torch.bfloat16 if it % 2 else torch.float32
            n = 8 * (1000 + 37 * it) if it != 5 else (4 << 20)   # call 5 does not fit a slot -> NCCL path
            torch.manual_seed(100 * it + rank)
            shard = torch.randn(n, device=dev).to(dt)
            with torch.cuda.stream(side):        # a stream of its own, like FSDP's all-gather stream
                side.wait_stream(torch.cuda.current_stream())
                out = ag.allocate((n * world,), dtype=dt, device=dev)
                out[rank * n:(rank + 1) * n].copy_(shard)
                ag(output_tensor=out, input_tensor=out[rank * n:(rank + 1) * n], group=g)
            torch.cuda.current_stream().wait_stream(side)
            ref = torch.empty(n * world, dtype=dt, device=dev)
            dist.all_gather_into_tensor(ref, shard)
            assert torch.equal(out, ref), ("all_gather", it, rank)
            # reduce-scatter: [W, n] pieces, fp32 accumulation, AVG and SUM
            op = dist.ReduceOp.AVG if it % 3 else dist.ReduceOp.SUM
            grads = torch.randn(world * n, device=dev).to(dt)
            inp = rs.allocate((world * n,), dtype=dt, device=dev)
            inp.copy_(grads)
            res = rs.allocate((n,), dtype=dt, device=dev)
            rs(output_tensor=res, input_tensor=inp, group=g, op=op)
            both = [torch.empty_like(grads) for _ in range(world)]
            dist.all_gather(both, grads)
            want = sum(b[rank * n:(rank + 1) * n].float() for b in both)
            want = want / world if op == dist.ReduceOp.AVG else want
            tol = 1e-6 if dt == torch.float32 else 1e-2
            assert torch.allclose(res.float(), want, rtol=tol, atol=tol), ("reduce_scatter", it, rank)
        torch.cuda.synchronize()
        arena.check()
        assert arena.calls["nccl"] == 2 and arena.calls["all_gather"] == 8 and arena.calls["reduce_scatter"] == 8, arena.calls

        # the same kernels under FSDP2: training on peer memory equals training on NCCL
        a, eng_a = _train("p2p")
        assert eng_a.backend.peer_arenas and eng_a.backend.peer_arenas[0].calls["all_gather"] > 0
        assert eng_a.backend.peer_arenas[0].calls["reduce_scatter"] > 0
        for ar in eng_a.backend.peer_arenas:
            ar.check()
        b, eng_b = _train("nccl")
        assert not eng_b.backend.peer_arenas
        ta, tb = torch.tensor(a), torch.tensor(b)
        assert torch.allclose(ta, tb, rtol=2e-3, atol=2e-3), (ta, tb)
        assert kernels.comm_status() == (0, 0)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp_collectives_over_peer_memory_match_nccl():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker, args=(2, os.path.join(d, "rdzv"), d), nprocs=2, join=True, start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise
