"""Block-diffusion data and loss: mask rules, deterministic noise, packing, engine loss incl. the confidence term,
and sequence-parallel parity of the loss."""
import torch

from dist_utils import run_distributed
from torchturbo_b200.models.llada2_moe import BDDataset, block_diffusion_allow, build_bd_row, first_fit_decreasing, mask_noise
from torchturbo_b200.models.llada2_moe.bd import SEG_CLEAN, SEG_NOISY, SEG_PAD, BDSample

LLADA = dict(model_type="llada2_moe", vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
             num_attention_heads=4, num_key_value_heads=2, num_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
             moe_intermediate_size=16, first_k_dense_replace=1, pad_token_id=0, mask_token_id=1)


def test_noise_is_deterministic_and_confined():
    a, sa = mask_noise(64, 10, 50, seed=7)
    b, sb = mask_noise(64, 10, 50, seed=7)
    assert torch.equal(a, b) and sa == sb and 0.3 <= sa <= 0.8
    assert not a[:10].any() and not a[50:].any() and a.any()
    assert not torch.equal(a, mask_noise(64, 10, 50, seed=8)[0])


def test_block_mask_rules():
    # one sample, T = 8, blocks of 4: positions 0..7 noisy, 8..15 clean
    sample = torch.zeros(16, dtype=torch.long)
    seg = torch.tensor([SEG_NOISY] * 8 + [SEG_CLEAN] * 8)
    block = torch.tensor([0] * 4 + [1] * 4 + [0] * 4 + [1] * 4)
    allow = block_diffusion_allow(sample, seg, block)
    assert allow[0, :4].all() and not allow[0, 4:].any()                  # noisy block 0: itself only
    assert allow[5, 4:8].all() and allow[5, 8:12].all() and not allow[5, 12:].any() and not allow[5, :4].any()
    assert allow[9, 8:12].all() and not allow[9, 12:].any() and not allow[9, :8].any()   # clean block 0
    assert allow[13, 8:16].all()                                           # clean block 1 sees clean 0 and itself
    seg2 = seg.clone()
    seg2[7] = SEG_PAD
    assert not block_diffusion_allow(sample, seg2, block)[:, 7].any()      # padding is never a key


def test_row_layout_labels_and_packing():
    s = [BDSample(list(range(2, 12)), 3, index=0), BDSample(list(range(20, 26)), 2, index=1)]
    row = build_bd_row(s, 48, block_size=4, mask_id=1, pad_id=0)
    ids, lab, st = row["input_ids"][0], row["labels"][0], row["bd_structure"]
    assert ids.shape == (48,) and row["block_allow"].shape == (48, 48)
    assert torch.equal(ids[12:22], torch.arange(2, 12))                    # clean copy of sample 0 after its noisy half
    sup = lab != -100
    assert sup.any() and (ids[sup] == 1).all() and not sup[12:24].any()    # labels only on masked noisy positions
    assert torch.equal(lab[:12][sup[:12]], ids[12:24][sup[:12]])           # ... and they are the clean tokens
    allow = row["block_allow"]
    assert not allow[:24, 24:].any() and not allow[24:, :24].any()         # samples never see each other
    assert (st[0, 40:] == -1).all() and not allow[:, 40:].any()
    assert first_fit_decreasing([20, 9, 13, 40], 32, 4) == [[0, 1], [2]]   # 40 does not fit a row at all
    ds = BDDataset([{"input_ids": list(range(2, 2 + n)), "prompt_length": 3} for n in (20, 9, 13)], 32, mask_id=1, pad_id=0,
                   block_size=4, pack=True)
    assert len(ds) == 2 and torch.equal(ds[0]["input_ids"], ds[0]["input_ids"])


def _loss_worker(rank, world, sp, cap, out_dir, tag):
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": sp, "ep_size": 1},
                                                   "activation_checkpointing": {"enabled": False}, "diffusion": {"cap_lambda": cap}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(LLADA), "seed": 3})
    ds = BDDataset([{"input_ids": list(range(2, 30)), "prompt_length": 4}], 32, mask_id=1, pad_id=0, block_size=4)
    loss = eng.compute_diffusion_loss(model, dict(ds[0]), ga=1)
    loss.backward()
    g = sum(float(p.grad.detach().float().pow(2).sum()) if p.grad is not None and not hasattr(p.grad, "full_tensor")
            else float(p.grad.full_tensor().float().pow(2).sum()) if p.grad is not None else 0.0 for p in model.parameters())
    torch.save((float(loss), g), f"{out_dir}/{tag}_r{rank}.pt")


def test_diffusion_loss_single_and_sp(tmp_path):
    run_distributed(_loss_worker, 1, 1, 0.0, str(tmp_path), "a")
    l1, g1 = torch.load(tmp_path / "a_r0.pt")
    assert 3.0 < l1 < 7.0 and g1 > 0
    run_distributed(_loss_worker, 1, 1, 0.5, str(tmp_path), "b")
    assert torch.load(tmp_path / "b_r0.pt")[0] >= l1                       # the entropy term is non-negative
    run_distributed(_loss_worker, 2, 2, 0.0, str(tmp_path), "c")
    for r in range(2):
        assert abs(torch.load(tmp_path / f"c_r{r}.pt")[0] - l1) < 1e-4      # SP=2 reproduces the SP=1 mean


def test_block_diffusion_sampling_fills_blocks_in_order_and_stops_at_eos():
    """`generate`: every new block starts masked and ends committed, earlier blocks are frozen context, greedy sampling is
    repeatable, the result is cut at the first end-of-sequence token and never longer than asked."""
    from torchturbo_b200.models.llada2_moe.generate import generate
    from torchturbo_b200.models.registry import get_model

    cls = get_model("llada2_moe")
    torch.manual_seed(0)
    model = cls(cls.config_class(**{k: v for k, v in LLADA.items() if k != "model_type"}, torch_dtype="float32")).eval()
    prompt = torch.randint(2, 128, (11,))
    seen = []
    orig = model.forward

    def spy(*a, **kw):
        seen.append(kw["input_ids"][0].clone())
        return orig(*a, **kw)

    model.forward = spy
    out = generate(model, prompt, max_new_tokens=20, block_size=8, steps=4)
    model.forward = orig
    assert out.shape == (31,) and torch.equal(out[:11], prompt) and not bool((out == 1).any())      # no mask token left
    # three blocks of 8 (the last one cut to 4): the first call of a block sees it fully masked behind frozen context
    firsts = [s for s in seen if bool((s[-8:] == 1).all())]
    assert [int(s.numel()) for s in firsts] == [19, 27, 35]
    assert torch.equal(firsts[1][:19], out[:19]) and torch.equal(firsts[2][:27], out[:27])
    # inside a block the number of masked positions only goes down, by the per-step quota (8 -> 6 -> 4 -> 2 -> 0)
    first_block = [int((s[11:19] == 1).sum()) for s in seen if s.numel() == 19]
    assert first_block == [8, 6, 4, 2]
    assert torch.equal(generate(model, prompt, max_new_tokens=20, block_size=8, steps=4), out)       # greedy is repeatable
    eos = int(out[14])
    cut = generate(model, prompt, max_new_tokens=20, block_size=8, steps=4, eos_id=eos)
    assert cut.numel() <= 19 and int(cut[-1]) == eos and int((cut[11:] == eos).sum()) == 1
    torch.manual_seed(1)
    sampled = generate(model, prompt, max_new_tokens=8, block_size=8, steps=2, temperature=1.0)
    assert sampled.shape == (19,) and not bool((sampled == 1).any())
