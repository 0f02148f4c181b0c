"""Parity of this package's own modelling code and checkpoint format with Hugging Face `transformers`.

For every family whose HF class ships with the installed `transformers`:
  (a) a randomly initialised HF model is written with `save_pretrained`, loaded through `engine.build_model(path)`
      (weight converter: per-projection HF tensors -> fused `qkv_proj` / `gate_up_proj` / `weight1` / `weight2`), and
      must give the same logits and the same packed-batch loss in fp32;
  (b) the engine's HF export (`save_model(..., hf_export)`) is loaded by `AutoModelForCausalLM.from_pretrained` and must
      give the same logits again.
The reference gets the first property for free by subclassing the HF classes (models/qwen3_moe/model.py:19) and tests
its own modelling copies against them (tests/models/deepseek_v4/test_turbo_vs_base_precision.py)."""
import os

import pytest
import torch

from dist_utils import run_distributed

transformers = pytest.importorskip("transformers")

DENSE = dict(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=50000.0, tie_word_embeddings=False,
             max_position_embeddings=512, attention_bias=False)
MOE = dict(DENSE, moe_intermediate_size=48, num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
           mlp_only_layers=[], router_aux_loss_coef=0.0, output_router_logits=False)


LINEAR = dict(linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
              linear_num_value_heads=4, full_attention_interval=2)
MLA = dict(vocab_size=320, hidden_size=64, intermediate_size=160, moe_intermediate_size=48, num_hidden_layers=3,
           num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
           first_k_dense_replace=1, q_lora_rank=32, kv_lora_rank=24, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
           n_group=2, topk_group=1, max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False)


def _hf(kind):
    """(config, class) of the `transformers` model.  Attention runs in its eager form: the sparse-attention family
    builds its causal mask only there (with sdpa and no padding the mask is left to the kernel, and the indexer's
    selection then replaces it)."""
    from transformers.models.auto.configuration_auto import CONFIG_MAPPING

    if kind == "qwen3":
        cfg, cls = CONFIG_MAPPING["qwen3"](**DENSE), transformers.Qwen3ForCausalLM
    elif kind == "qwen3_moe":
        cfg, cls = CONFIG_MAPPING["qwen3_moe"](**MOE), transformers.Qwen3MoeForCausalLM
    elif kind == "qwen3_5_moe_text":
        base = {k: v for k, v in DENSE.items() if k not in ("rope_theta", "attention_bias")}
        cfg = CONFIG_MAPPING[kind](**dict(base, num_hidden_layers=4), **LINEAR, moe_intermediate_size=48,
                                   shared_expert_intermediate_size=48, num_experts=8, num_experts_per_tok=2)
        cls = transformers.Qwen3_5MoeForCausalLM
    elif kind == "glm_moe_dsa":
        # eight index heads: with two, a quarter of all index scores are exactly zero after the ReLU, and among tied keys
        # `torch.topk` (transformers) and this package's stable order (the same under any slicing of the queries) may differ
        cfg = CONFIG_MAPPING[kind](**MLA, index_n_heads=8, index_head_dim=16, index_topk=8)
        cls = transformers.GlmMoeDsaForCausalLM
    else:
        raise KeyError(kind)
    cfg._attn_implementation = "eager"
    return cfg, cls


def _engine():
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine

    return TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "activation_checkpointing": {"enabled": False},
                                                    "checkpoint": {"hf_export": "every"}}))


def _hf_logits(model, ids, lens):
    """Packed row through the HF model: one forward per document (position ids restart, no cross-document attention)."""
    outs, s = [], 0
    with torch.no_grad():
        for n in lens:
            outs.append(model(input_ids=ids[:, s:s + n]).logits.float())
            s += n
    return torch.cat(outs, dim=1)


def _batch(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    ids = torch.randint(0, vocab, (1, T), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens])[None]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    labels = ids.clone()
    labels[0, cu[:-1].long()] = -100
    return dict(input_ids=ids, position_ids=pos, labels=labels, cu_seq_lens_q=cu, cu_seq_lens_k=cu,
                max_length_q=max(lens), max_length_k=max(lens))


def _w_parity(rank, world, kind, root):
    torch.manual_seed(0)
    cfg, cls = _hf(kind)
    hf = cls(cfg).float().eval()
    with torch.no_grad():        # norm weights and biases away from their constant initial values
        for p in hf.parameters():
            if p.ndim == 1:
                p.add_(torch.randn_like(p) * 0.1)
    src = os.path.join(root, "hf_src")
    hf.save_pretrained(src, safe_serialization=True)
    lens = [23, 9, 16]
    batch = _batch(cfg.vocab_size, lens)
    ref_logits = _hf_logits(hf, batch["input_ids"], lens)
    # ---- (a) HF checkpoint -> this engine
    eng = _engine()
    model = eng.build_model(src)
    model.eval()
    with torch.no_grad():
        out = model(**{k: v for k, v in batch.items() if k != "labels"})
    ours = out["logits"].float().reshape(1, -1, cfg.vocab_size)
    err = (ours - ref_logits).abs().max().item()
    assert err < 1e-4, f"{kind}: logits differ from transformers by {err}"
    # packed loss: mean CE over the targets that stay inside their document
    model.train()
    loss = float(eng.compute_loss(model, dict(batch)))
    tgt, lg = [], []
    s = 0
    for n in lens:
        lg.append(ref_logits[0, s:s + n - 1])
        tgt.append(batch["input_ids"][0, s + 1:s + n])
        s += n
    ref_loss = float(torch.nn.functional.cross_entropy(torch.cat(lg), torch.cat(tgt)))
    assert abs(loss - ref_loss) < 1e-4, (kind, loss, ref_loss)
    # ---- (b) this engine's HF export -> transformers
    ckpt = os.path.join(root, "checkpoint-1")
    eng.save_model(model, ckpt, final=True)
    back = transformers.AutoModelForCausalLM.from_pretrained(os.path.join(ckpt, "huggingface"), dtype=torch.float32,
                                                                attn_implementation="eager").eval()
    sd_a, sd_b = hf.state_dict(), back.state_dict()
    assert set(sd_a) == set(sd_b), sorted(set(sd_a) ^ set(sd_b))[:8]
    # the export is written in bf16 (the training compute dtype): every tensor must be the bf16 rounding of its source,
    # in the source's own name and layout, so the logits equal those of the source model with bf16-rounded weights
    for k in sd_a:
        assert torch.equal(sd_b[k].float(), sd_a[k].bfloat16().float()), k
    hf.load_state_dict({k: v.bfloat16().float() for k, v in sd_a.items()})
    err = (_hf_logits(back, batch["input_ids"], lens) - _hf_logits(hf, batch["input_ids"], lens)).abs().max().item()
    assert err < 1e-5, f"{kind}: exported checkpoint differs from the (bf16-rounded) source by {err}"


@pytest.mark.parametrize("kind", ["qwen3", "qwen3_moe", "qwen3_5_moe_text", "glm_moe_dsa"])
def test_logits_loss_and_export_match_transformers(tmp_path, kind):
    run_distributed(_w_parity, 1, kind, str(tmp_path), timeout=400)


def _fuse_expert_files(src):
    """Rewrite the per-expert tensors of a checkpoint as the fused 3-D tensors that published Qwen3.5-MoE checkpoints
    carry: `experts.gate_up_proj [E, 2F, H]`, `experts.down_proj [E, H, F]`."""
    import re

    from safetensors.torch import load_file, save_file

    path = os.path.join(src, "model.safetensors")
    sd = {k: v.clone() for k, v in load_file(path).items()}     # the file is rewritten below: no memory-mapped views
    groups = {}
    for k in list(sd):
        m = re.match(r"(.*\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$", k)
        if m:
            groups.setdefault(m.group(1), {}).setdefault(m.group(3), {})[int(m.group(2))] = sd.pop(k)
    for pre, g in groups.items():
        n = len(g["gate_proj"])
        sd[f"{pre}.gate_up_proj"] = torch.stack([torch.cat([g["gate_proj"][e], g["up_proj"][e]], 0) for e in range(n)])
        sd[f"{pre}.down_proj"] = torch.stack([g["down_proj"][e] for e in range(n)])
    save_file(sd, path, metadata={"format": "pt"})
    return sd


def _w_fused_layout(rank, world, root):
    torch.manual_seed(0)
    cfg, cls = _hf("qwen3_5_moe_text")
    hf = cls(cfg).float().eval()
    src = os.path.join(root, "hf_src")
    hf.save_pretrained(src, safe_serialization=True)
    fused = _fuse_expert_files(src)
    assert any(k.endswith("experts.gate_up_proj") for k in fused)
    lens = [19, 14]
    batch = _batch(cfg.vocab_size, lens)
    ref_logits = _hf_logits(hf, batch["input_ids"], lens)
    eng = _engine()
    model = eng.build_model(src)
    model.eval()
    with torch.no_grad():
        out = model(**{k: v for k, v in batch.items() if k != "labels"})
    err = (out["logits"].float().reshape(1, -1, cfg.vocab_size) - ref_logits).abs().max().item()
    assert err < 1e-4, f"fused expert layout: logits differ from transformers by {err}"
    ckpt = os.path.join(root, "checkpoint-1")
    eng.save_model(model, ckpt, final=True)
    from safetensors import safe_open

    got = {}
    hf_dir = os.path.join(ckpt, "huggingface")
    for f in sorted(os.listdir(hf_dir)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(hf_dir, f), "pt") as sf:
                for k in sf.keys():
                    got[k] = sf.get_tensor(k)
    assert set(got) == set(fused), sorted(set(got) ^ set(fused))[:8]
    for k, v in fused.items():
        assert got[k].shape == v.shape and torch.equal(got[k].float(), v.bfloat16().float()), k


def test_fused_expert_checkpoint_layout_round_trip(tmp_path):
    """Checkpoints with 3-D fused expert tensors load into the engine's `[E*H, 2F]` / `[E*F, H]` parameters (each
    expert transposed) and are exported in the same fused layout and names."""
    run_distributed(_w_fused_layout, 1, str(tmp_path), timeout=400)


# ---- vision-language families: tower, placeholder fusion, multimodal rotary positions, DeepStack --------------------
VIS = dict(depth=2, hidden_size=32, num_heads=4, intermediate_size=48, patch_size=2, temporal_patch_size=2, in_channels=3,
           spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=16)
IMG, VSTART = 300, 301


def _hf_vlm(kind):
    from transformers.models.auto.configuration_auto import CONFIG_MAPPING

    text = {k: v for k, v in DENSE.items() if k not in ("rope_theta", "attention_bias", "tie_word_embeddings")}
    text["num_hidden_layers"] = 4
    if kind in ("qwen3_5", "qwen3_5_moe"):
        text.update(LINEAR, rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                             "mrope_section": [2, 1, 1], "mrope_interleaved": True})
        if kind == "qwen3_5_moe":
            text.pop("intermediate_size")
            text.update(moe_intermediate_size=48, shared_expert_intermediate_size=48, num_experts=8, num_experts_per_tok=2)
        vis = dict(VIS)
        cls = transformers.Qwen3_5ForConditionalGeneration if kind == "qwen3_5" else transformers.Qwen3_5MoeForConditionalGeneration
    else:
        text.update(rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2],
                                     "mrope_interleaved": True})
        vis, cls = dict(VIS, deepstack_visual_indexes=[0, 1]), transformers.Qwen3VLForConditionalGeneration
    cfg = CONFIG_MAPPING[kind](text_config=text, vision_config=vis, image_token_id=IMG, video_token_id=302,
                               vision_start_token_id=VSTART, tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    return cfg, cls


def _published_key(k: str) -> str:
    """`save_pretrained` of the installed transformers applies its load-time renaming in reverse once too often for
    these classes (`model.language_model.language_model.*`, `model.language_model.visual.*`); published checkpoints
    have `model.language_model.*` and `model.visual.*`."""
    import re

    k = re.sub(r"^model\.(language_model\.)+visual\.", "model.visual.", k)
    return k if k.startswith("model.visual.") else re.sub(r"^model\.(language_model\.)+", "model.language_model.", k)


def _w_vlm(rank, world, kind, root):
    from safetensors import safe_open
    from safetensors.torch import load_file, save_file

    torch.manual_seed(0)
    cfg, cls = _hf_vlm(kind)
    hf = cls(cfg).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim == 1:
                p.add_(torch.randn_like(p) * 0.1)
    src = os.path.join(root, "hf_src")
    hf.save_pretrained(src, safe_serialization=True)
    fp = os.path.join(src, "model.safetensors")
    published = {_published_key(k): v.clone() for k, v in load_file(fp).items()}
    save_file(published, fp, metadata={"format": "pt"})
    grid = torch.tensor([[1, 4, 4], [1, 2, 6]])                      # two images: 16 and 12 patches -> 4 and 3 rows
    pixels = torch.randn(int(grid.prod(-1).sum()), 3 * 2 * 2 * 2)
    T = 40
    ids = torch.randint(0, 290, (1, T))
    ids[0, 3], ids[0, 20] = VSTART, VSTART
    ids[0, 4:8], ids[0, 21:24] = IMG, IMG
    mm = (ids == IMG).int()
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=mm).logits.float()
        pos = hf.model.get_rope_index(ids, mm_token_type_ids=mm, image_grid_thw=grid)[0]          # [3, 1, T]
        tower_ref = hf.model.visual(pixels, grid_thw=grid).pooler_output
    eng = _engine()
    model = eng.build_model(src)
    model.eval()
    cu = torch.tensor([0, T], dtype=torch.int32)
    with torch.no_grad():
        tower = model.model.visual(pixels, grid_thw=grid)
        out = model(input_ids=ids, position_ids=pos, pixel_values=pixels, image_grid_thw=grid, cu_seq_lens_q=cu,
                    cu_seq_lens_k=cu, max_length_q=T, max_length_k=T)
    assert (tower - tower_ref).abs().max().item() < 1e-5, f"{kind}: vision tower differs from transformers"
    err = (out["logits"].float().reshape(1, T, -1) - ref).abs().max().item()
    assert err < 1e-4, f"{kind}: logits with images differ from transformers by {err}"
    # export: same names, same (bf16-rounded) tensors as the published layout of the source
    ckpt = os.path.join(root, "checkpoint-1")
    eng.save_model(model, ckpt, final=True)
    got = {}
    hf_dir = os.path.join(ckpt, "huggingface")
    for f in sorted(os.listdir(hf_dir)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(hf_dir, f), "pt") as sf:
                for k in sf.keys():
                    got[k] = sf.get_tensor(k)
    assert set(got) == set(published), sorted(set(got) ^ set(published))[:8]
    for k, v in published.items():
        assert got[k].shape == v.shape and torch.equal(got[k].float(), v.bfloat16().float()), k


@pytest.mark.parametrize("kind", ["qwen3_5", "qwen3_5_moe", "qwen3_vl"])
def test_vision_language_logits_and_export_match_transformers(tmp_path, kind):
    run_distributed(_w_vlm, 1, kind, str(tmp_path), timeout=400)


def _w_kimi(rank, world, root):
    """`kimi_k25` on a checkpoint laid out like the published one (`language_model.*`, `vision_tower.*`,
    `mm_projector.*`): the decoder must equal `transformers.DeepseekV3ForCausalLM` on text, and a row with media must
    run through MoonViT and the projector."""
    import json

    from safetensors.torch import load_file, save_file
    from transformers.models.auto.configuration_auto import CONFIG_MAPPING

    from torchturbo_b200.models.kimi_k25.vision import MoonViT, MoonViTConfig, PatchMergerMLP, init_moonvit

    torch.manual_seed(0)
    cfg = CONFIG_MAPPING["deepseek_v3"](**MLA)
    cfg._attn_implementation = "eager"
    hf = transformers.DeepseekV3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim == 1:
                p.add_(torch.randn_like(p) * 0.1)
    lm_dir, src = os.path.join(root, "lm"), os.path.join(root, "kimi")
    hf.save_pretrained(lm_dir, safe_serialization=True)
    sd = {"language_model." + k: v.clone() for k, v in load_file(os.path.join(lm_dir, "model.safetensors")).items()}
    vcfg = dict(patch_size=14, init_pos_emb_height=6, init_pos_emb_width=6, init_pos_emb_time=4, vt_num_attention_heads=4,
                vt_num_hidden_layers=2, vt_hidden_size=64, vt_intermediate_size=96, merge_kernel_size=[2, 2],
                text_hidden_size=MLA["hidden_size"])
    vc = MoonViTConfig(**vcfg)
    tower, proj = MoonViT(vc, torch.float32), PatchMergerMLP(vc, torch.float32)
    init_moonvit(tower, proj, 0.05)
    sd.update({"vision_tower." + k: v.clone() for k, v in tower.state_dict().items()})
    sd.update({"mm_projector." + k: v.clone() for k, v in proj.state_dict().items()})
    os.makedirs(src)
    save_file(sd, os.path.join(src, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(lm_dir, "config.json")) as f:
        text_cfg = json.load(f)
    with open(os.path.join(src, "config.json"), "w") as f:
        json.dump({"model_type": "kimi_k25", "text_config": text_cfg, "vision_config": vcfg, "media_placeholder_token_id": 300}, f)
    T = 24
    ids = torch.randint(0, 290, (1, T))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits.float()
    eng = _engine()
    model = eng.build_model(src)
    model.eval()
    for k, v in tower.state_dict().items():
        assert torch.equal(model.vision_tower.state_dict()[k], v), k          # the tower was loaded by name
    cu = torch.tensor([0, T], dtype=torch.int32)
    kw = dict(position_ids=torch.arange(T)[None], cu_seq_lens_q=cu, cu_seq_lens_k=cu, max_length_q=T, max_length_k=T)
    with torch.no_grad():
        out = model(input_ids=ids, **kw)["logits"].float().reshape(1, T, -1)
    err = (out - ref).abs().max().item()
    assert err < 1e-4, f"kimi_k25 decoder differs from transformers.DeepseekV3ForCausalLM by {err}"
    # one 4x4-patch image -> 4 media tokens
    ids[0, 5:9] = 300
    with torch.no_grad():
        with_img = model(input_ids=ids, pixel_values=torch.randn(16, 3, 14, 14), grid_thws=torch.tensor([[1, 4, 4]]), **kw)["logits"]
    assert torch.isfinite(with_img).all() and (with_img.float().reshape(1, T, -1)[0, 9:] - out[0, 9:]).abs().max() > 1e-4


def test_kimi_k25_decoder_matches_transformers_and_tower_loads_by_name(tmp_path):
    run_distributed(_w_kimi, 1, str(tmp_path), timeout=400)
