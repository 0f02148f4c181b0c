"""Direct preference optimisation on packed rows (`loops/dpo.py`): preference losses against hand formulas, LD-DPO
token weights, segment sums over a sequence-parallel shard, a full step on a tiny model, and SP-2 == SP-1."""
import math

import pytest
import torch
import torch.nn.functional as F

from dist_utils import run_distributed
from torchturbo_b200.loops.dpo import DPOConfig, dpo_loss, segment_sums, segment_token_weights

IGN = -100


def test_preference_losses_match_their_formulas():
    pol = torch.tensor([-10.0, -12.0, -14.0, -11.0])        # chosen 0, 1; rejected 0, 1
    ref = torch.tensor([-11.0, -12.5, -13.0, -11.5])
    counts = torch.tensor([5.0, 4.0, 5.0, 2.0])
    h = (pol[:2] - pol[2:]) - (ref[:2] - ref[2:])
    loss, m = dpo_loss(pol, ref, counts, DPOConfig(beta=0.5))
    assert torch.allclose(loss, (-F.logsigmoid(0.5 * h)).mean())
    assert torch.allclose(m["rewards/chosen"], (0.5 * (pol[:2] - ref[:2])).mean())
    assert float(m["rewards/accuracies"]) == 0.5             # pair 0: chosen gains more than rejected; pair 1: the same
    smooth, _ = dpo_loss(pol, ref, counts, DPOConfig(beta=0.5, label_smoothing=0.2))
    assert torch.allclose(smooth, (-0.8 * F.logsigmoid(0.5 * h) - 0.2 * F.logsigmoid(-0.5 * h)).mean())
    hinge, _ = dpo_loss(pol, ref, counts, DPOConfig(beta=0.5, loss_type="hinge"))
    assert torch.allclose(hinge, torch.relu(1 - 0.5 * h).mean())
    ipo, _ = dpo_loss(pol, ref, counts, DPOConfig(beta=0.5, loss_type="ipo"))
    hn = (pol / counts)[:2] - (pol / counts)[2:] - ((ref / counts)[:2] - (ref / counts)[2:])   # length-normalised
    assert torch.allclose(ipo, ((hn - 1.0) ** 2).mean())
    sft, _ = dpo_loss(pol, ref, counts, DPOConfig(beta=0.5, sft_alpha=0.3))
    assert torch.allclose(sft, (-F.logsigmoid(0.5 * h) - 0.3 * pol[:2] / counts[:2]).mean())
    with pytest.raises(ValueError):
        dpo_loss(pol, ref, counts, DPOConfig(loss_type="nope"))


def test_ld_weights_discount_only_the_tail_of_the_longer_answer():
    # pair 0: chosen has 3 targets, rejected 5; pair 1: 4 and 2
    lab = torch.full((1, 24), IGN)
    cu = torch.tensor([0, 6, 12, 18, 24])                    # chosen 0, chosen 1, rejected 0, rejected 1
    lab[0, 2:5] = 7
    lab[0, 7:11] = 7
    lab[0, 13:18] = 7
    lab[0, 20:22] = 7
    w = segment_token_weights(lab, cu, DPOConfig(ld_alpha=0.25))
    assert w[2:5].tolist() == [1, 1, 1] and w[13:18].tolist() == [1, 1, 1, 0.25, 0.25]
    assert w[7:11].tolist() == [1, 1, 0.25, 0.25] and w[20:22].tolist() == [1, 1]
    assert float(w[lab[0] == IGN].sum()) == 0.0
    plain = segment_token_weights(lab, cu, DPOConfig())
    assert torch.equal(plain, (lab[0] != IGN).float())


def test_segment_sums_of_a_shard_add_up_to_the_row():
    v = torch.arange(20.0)
    offs = [0, 7, 7, 15, 20]
    whole = segment_sums(v, offs, 0, 20)
    assert whole.tolist() == [21.0, 0.0, sum(range(7, 15)), sum(range(15, 20))]
    parts = segment_sums(v[:10], offs, 0, 10) + segment_sums(v[10:], offs, 10, 20)
    assert torch.equal(parts, whole)


DENSE = dict(model_type="qwen3", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
             intermediate_size=128, vocab_size=256, tie_word_embeddings=False)


def _pair_row(seed):
    g = torch.Generator().manual_seed(seed)
    segs, labels = [], []
    for n_prompt, n_ans in ((5, 7), (4, 6), (5, 9), (4, 5)):        # chosen 0, chosen 1, rejected 0, rejected 1 (32 + 13 = 45 -> pad 48)
        ids = torch.randint(1, 256, (n_prompt + n_ans,), generator=g)
        segs.append(ids)
        labels.append(torch.cat((torch.full((n_prompt,), IGN), ids[n_prompt:])))
    ids, lab = torch.cat(segs), torch.cat(labels)
    cu = torch.tensor([0, 12, 22, 36, 45], dtype=torch.int32)
    pad = 48 - ids.numel()
    ids, lab = F.pad(ids, (0, pad)), F.pad(lab, (0, pad), value=IGN)
    pos = torch.cat([torch.arange(b - a) for a, b in zip(cu[:-1].tolist(), cu[1:].tolist())] + [torch.arange(pad)])
    return {"input_ids": ids[None], "labels": lab[None], "position_ids": pos[None], "cu_seq_lens_q": cu, "cu_seq_lens_k": cu.clone(),
            "max_length_q": 14, "max_length_k": 14}


def _w_dpo(rank, world, sp, out):
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops.dpo import build_reference_model, dpo_step, sequence_logps

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": sp, "ep_size": 1},
                                                   "activation_checkpointing": {"enabled": False}}))
    policy = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(DENSE), "seed": 0})
    reference = build_reference_model(eng, policy=policy, init_kwargs={"config": dict(DENSE), "seed": 1})
    assert not any(p.requires_grad for p in reference.parameters())
    cfg = DPOConfig(beta=0.5)
    batch = _pair_row(3)
    pol, counts = sequence_logps(eng, policy, batch, cfg, grad=False)
    ref, _ = sequence_logps(eng, reference, batch, DPOConfig(0.5), grad=False)
    assert counts.tolist() == [7.0, 6.0, 9.0, 5.0]               # one target per answer token (the first is predicted from the prompt)
    opt = eng.prepare_optimizer(policy, OptimizerClassPlan(torch.optim.AdamW, lr=5e-3, weight_decay=0.0))
    hist = []
    for _ in range(4):
        loss, gn, m = dpo_step(eng, policy, reference, opt, batch, cfg)
        hist.append([float(loss), float(gn), float(m["rewards/margins"])])
    # same policy and reference at the start: the first loss is log 2
    assert torch.allclose(pol, ref, atol=1e-5) and abs(hist[0][0] - math.log(2)) < 1e-4
    assert hist[-1][0] < hist[0][0] and hist[-1][2] > hist[0][2]
    if rank == 0:
        torch.save({"pol": pol, "hist": torch.tensor(hist)}, out)


def test_dpo_steps_reduce_the_loss_and_sequence_parallel_matches(tmp_path):
    run_distributed(_w_dpo, 2, 1, str(tmp_path / "sp1.pt"), timeout=600)
    run_distributed(_w_dpo, 2, 2, str(tmp_path / "sp2.pt"), timeout=600)
    a, b = torch.load(tmp_path / "sp1.pt"), torch.load(tmp_path / "sp2.pt")
    assert torch.allclose(a["pol"], b["pol"], rtol=1e-4, atol=1e-4)
    assert torch.allclose(a["hist"], b["hist"], rtol=2e-3, atol=2e-4), (a["hist"], b["hist"])
