"""Every registered model family builds at toy size on CPU, runs a packed forward/backward, and keeps the
packed-sequence isolation property (a token never sees another document)."""
import pytest
import torch

from torchturbo_b200.models.registry import get_model, list_models

TEXT = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4, torch_dtype="float32")
VISION = dict(depth=1, hidden_size=16, num_heads=2, intermediate_size=32, patch_size=2, temporal_patch_size=1)
QWEN35 = dict(TEXT, num_attention_heads=2, num_key_value_heads=1, head_dim=16, linear_key_head_dim=8, linear_value_head_dim=8,
              linear_num_key_heads=2, linear_num_value_heads=4, mrope_section=(1, 1, 0), mtp_num_hidden_layers=1)
QMOE = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, shared_expert_intermediate_size=16)
MLA = dict(kv_lora_rank=16, qk_rope_head_dim=4, qk_nope_head_dim=8, v_head_dim=8)
DSV3 = dict(TEXT, moe_intermediate_size=16, num_hidden_layers=3, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
            first_k_dense_replace=1, q_lora_rank=24, num_nextn_predict_layers=1, **MLA)


def _build(model_type):
    cls = get_model(model_type)
    if model_type == "qwen3_5":
        cfg = cls.config_class(text_config=QWEN35, vision_config=VISION, image_token_id=5)
    elif model_type == "qwen3_5_moe":
        cfg = cls.config_class(text_config=dict(QWEN35, **QMOE), vision_config=VISION, image_token_id=5)
    elif model_type == "qwen3_5_moe_text":
        cfg = cls.config_class(**dict(QWEN35, **QMOE))
    elif model_type == "bailing_hybrid":
        cfg = cls.config_class(**dict(TEXT, num_hidden_layers=5, head_dim=8, num_experts=8, num_experts_per_tok=2, n_group=2,
                                      topk_group=1, moe_intermediate_size=16, moe_shared_expert_intermediate_size=16,
                                      layer_group_size=3, num_nextn_predict_layers=1, pad_token_id=0,
                                      gated_attention_proj_granularity_type="head_wise", **MLA))
    elif model_type == "bailing_moe_v3_vl":
        tc = dict(TEXT, num_hidden_layers=5, head_dim=8, num_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
                  moe_intermediate_size=16, moe_shared_expert_intermediate_size=16, layer_group_size=3,
                  num_nextn_predict_layers=1, pad_token_id=0, **MLA)
        cfg = cls.config_class(text_config=tc, vision_config=VISION, image_patch_token=5, video_patch_token=4)
    elif model_type == "kimi_k25":
        cfg = cls.config_class(text_config=DSV3, media_placeholder_token_id=5,
                               vision_config=dict(vt_num_hidden_layers=1, vt_hidden_size=16, vt_num_attention_heads=2,
                                                  vt_intermediate_size=32, patch_size=2, merge_kernel_size=(2, 2)))
    elif model_type == "deepseek_v4":
        cfg = cls.config_class(**dict(TEXT, moe_intermediate_size=16, num_hidden_layers=3, n_routed_experts=8, num_experts_per_tok=2,
                                      q_lora_rank=16, qk_rope_head_dim=4, qk_nope_head_dim=12, o_groups=2, o_lora_rank=8,
                                      sliding_window=4, compress_ratios=[1, 4, 2], index_n_heads=2, index_head_dim=8, index_topk=2,
                                      hc_mult=2, hc_sinkhorn_iters=3, swiglu_limit=7.0, num_hash_layers=1, num_mtp_layers=1))
    elif model_type == "qwen4_exp":
        tc = dict(QWEN35, **QMOE, hc_count=2, hc_lowrank=8, ple_layer_ids=[1, 2], ple_embed_dim=16, ple_conv_kernel_size=2,
                  ngram_size=3, heads_per_ngram=2, ngram_vocab_size_base=50, make_ngram_vocab_size_divisible_by=8,
                  indexer_n_heads=2, indexer_head_dim=16, indexer_budget=4, indexer_compress_ratio=2, eos_token_id=0)
        tc.pop("mtp_num_hidden_layers")
        cfg = cls.config_class(text_config=tc, vision_config=VISION, image_token_id=5)
    elif model_type == "glm_moe_dsa":
        cfg = cls.config_class(**dict(DSV3, num_hidden_layers=4, n_group=1, num_nextn_predict_layers=0, index_topk=6,
                                      index_head_dim=8, index_n_heads=2, index_topk_freq=2, index_skip_topk_offset=1,
                                      mlp_layer_types=["dense", "sparse", "sparse", "sparse"]))
    else:
        pytest.skip(f"no toy config for {model_type}")
    torch.manual_seed(0)
    return cls, cls(cfg)


def _batch(vlm: bool, media_key="image_grid_thw"):
    ids = torch.randint(6, 128, (1, 24))
    b = dict(input_ids=ids, cu_seq_lens_q=torch.tensor([0, 10, 24], dtype=torch.int32), max_length_q=14)
    if vlm:
        ids[0, 3:7] = 5
        b["pixel_values"] = torch.randn(16, 3 * 1 * 2 * 2)
        b[media_key] = torch.tensor([[1, 4, 4]])
    return b


FAMILIES = ["qwen3_5", "qwen3_5_moe", "qwen3_5_moe_text", "bailing_hybrid", "bailing_moe_v3_vl", "kimi_k25", "glm_moe_dsa",
            "deepseek_v4", "qwen4_exp"]


def test_all_families_registered():
    assert set(FAMILIES + ["qwen3", "qwen3_moe", "qwen3_vl", "llada2_moe"]) <= set(list_models())


@pytest.mark.parametrize("model_type", FAMILIES)
def test_family_forward_backward_and_isolation(model_type):
    cls, m = _build(model_type)
    m.train()
    vlm = model_type in ("qwen3_5", "qwen3_5_moe", "kimi_k25", "bailing_moe_v3_vl", "qwen4_exp")
    b = _batch(vlm, "grid_thws" if model_type == "kimi_k25" else "image_grid_thw")
    out = m(**b)
    assert out.logits.shape == (1, 24, 128) and torch.isfinite(out.logits).all()
    loss = out.logits.float().pow(2).mean()
    for h in out.get("mtp_logits") or ():
        loss = loss + h.float().pow(2).mean()
    loss.backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None and p.requires_grad and ".indexer." not in n]
    assert not missing, missing
    # document isolation: changing the second document leaves the first document's logits untouched
    m.eval()
    with torch.no_grad():
        base = m(**b).logits
        b2 = dict(b, input_ids=b["input_ids"].clone())
        b2["input_ids"][0, 15:20] = torch.randint(6, 128, (5,))
        other = m(**b2).logits
    assert torch.allclose(base[0, :10], other[0, :10], atol=1e-5)
    assert not torch.allclose(base[0, 10:], other[0, 10:], atol=1e-5)
    # the plan names real modules and the converter maps every parameter to a checkpoint name
    plan = cls.get_default_parallel_plan()
    names = {n for n, _ in m.named_modules()}
    from torchturbo_b200.engine.utils import match_fqn

    for pat in plan.plan:
        if pat.startswith("mtp") and getattr(m, "mtp", None) is None:
            continue
        assert any(match_fqn(pat, n) for n in names), pat
    conv = m.get_weight_converter({})
    for n, _ in m.named_parameters():
        r = conv.load_recipe(n)
        assert r is None or all(isinstance(s, str) and s for s in r.sources)


def test_mrope_axis_assignment_and_roll():
    from torchturbo_b200.models.modules.hybrid import MRotaryEmbedding, roll_left_in_sequences

    rot = MRotaryEmbedding(16, 10000.0, mrope_section=(4, 2, 2), interleaved=True)
    assert rot.axis_of_pair(8, "cpu").tolist() == [0, 1, 2, 0, 1, 2, 0, 0]
    rot2 = MRotaryEmbedding(16, 10000.0, mrope_section=(4, 2, 2), interleaved=False)
    assert rot2.axis_of_pair(8, "cpu").tolist() == [0, 0, 0, 0, 1, 1, 2, 2]
    pos = torch.stack([torch.arange(5), torch.arange(5) * 2, torch.arange(5) * 3])
    cos, _ = rot(pos)
    cos_t, _ = rot(torch.arange(5))
    assert torch.allclose(cos[:, 0], cos_t[:, 0]) and not torch.allclose(cos[:, 1], cos_t[:, 1])
    ids = torch.arange(1, 9).view(1, -1)
    assert roll_left_in_sequences(ids, [0, 3, 8], fill=0)[0].tolist() == [2, 3, 0, 5, 6, 7, 8, 0]


def test_sparse_attention_ops():
    from torchturbo_b200.ops import ops
    from torchturbo_b200.ops.providers import native as N

    torch.manual_seed(0)
    T, H, D = 40, 4, 8
    q, k, v = torch.randn(T, H, D), torch.randn(T, 2, D), torch.randn(T, 2, D)
    cu = torch.tensor([0, 15, 40], dtype=torch.int32)
    qi, ki, w = torch.randn(T, 3, 6), torch.randn(T, 6), torch.rand(T, 3)
    full = ops.lightning_indexer(qi, ki, w, 64, cu_seqlens=cu)
    assert torch.allclose(ops.sparse_attention(q, k, v, full), N.attention_ref(q, k, v, cu, causal=True), atol=1e-5)
    top = ops.lightning_indexer(qi, ki, w, 4, cu_seqlens=cu)
    assert top.shape == (T, 4) and int(top[15, 0]) == 15 and (top[15, 1:] == -1).all()
    assert ((top < 0) | ((top >= 15) == (torch.arange(T)[:, None] >= 15))).all()          # never across documents
    half = ops.lightning_indexer(qi[20:], ki, w[20:], 4, cu_seqlens=cu, q_offset=20)       # an SP shard of the queries
    assert torch.equal(half, top[20:])
    o = ops.sparse_flash_mla(q, k[:, 0], None, None, None, torch.zeros(H), D ** -0.5, 1, 3, cu_seq_lens_q=cu)
    assert o.shape == (T, H, D) and torch.isfinite(o).all()


def test_deepseek_v4_indexer_kl_loss_trains_the_indexer():
    """Off by default: the indexer only selects (no gradient).  With `dsa_indexer_loss_coeff > 0` the KL term between
    the main attention over the selected compressed rows and the indexer's softmax reaches the indexer's parameters
    and nothing else changes in the reported loss."""
    import torch.nn.functional as F

    cls = get_model("deepseek_v4")
    kw = dict(TEXT, moe_intermediate_size=16, num_hidden_layers=2, n_routed_experts=8, num_experts_per_tok=2, q_lora_rank=16,
              qk_rope_head_dim=4, qk_nope_head_dim=12, o_groups=2, o_lora_rank=8, sliding_window=4, compress_ratios=[1, 4],
              index_n_heads=2, index_head_dim=8, index_topk=2, hc_mult=2, hc_sinkhorn_iters=3)
    b = _batch(False)
    losses, grads = {}, {}
    for coeff in (0.0, 0.5):
        torch.manual_seed(0)
        m = cls(cls.config_class(**kw, dsa_indexer_loss_coeff=coeff)).float().train()
        loss = m(**b).logits.float().pow(2).mean()
        loss.backward()
        losses[coeff] = loss.item()
        idx_params = {n: p for n, p in m.named_parameters() if ".indexer." in n}
        assert idx_params
        grads[coeff] = {n: (None if p.grad is None else p.grad.abs().sum().item()) for n, p in idx_params.items()}
        attn = [mod for mod in m.modules() if getattr(mod, "indexer", None) is not None][0]
        if coeff:
            assert attn.last_indexer_loss is not None and attn.last_indexer_loss.item() >= 0
        else:
            assert attn.last_indexer_loss is None
    assert losses[0.0] == pytest.approx(losses[0.5], rel=1e-6)          # the reported LM loss is unchanged
    assert all(g in (None, 0.0) for g in grads[0.0].values())
    assert any(g for g in grads[0.5].values() if g)

    # the formula, against a direct restatement on small tensors
    torch.manual_seed(1)
    t = torch.rand(5, 3)
    s = torch.randn(5, 3)
    valid = torch.tensor([[1, 1, 0], [1, 0, 0], [0, 0, 0], [1, 1, 1], [1, 1, 1]], dtype=torch.bool)
    p = torch.softmax(s.masked_fill(~valid, torch.finfo(torch.float32).min), -1).masked_fill(~valid, 0)
    tt = F.normalize(t.masked_fill(~valid, 0), p=1, dim=-1)
    want = F.kl_div((p + 1e-10).log(), tt, reduction="none").sum() / valid.any(-1).sum()
    got = torch.where(tt > 0, tt * (tt.clamp_min(1e-30).log() - (p + 1e-10).log()), torch.zeros_like(tt)).sum() / valid.any(-1).sum()
    assert torch.allclose(want, got, atol=1e-6)
