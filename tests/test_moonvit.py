"""MoonViT (Kimi-K2.5 vision tower) and its patch-merger projector against a plain fp32 torch formulation written from
the published description (complex-number 2-D rotary embedding, per-medium full attention, temporal pooling), and the
module tree against the parameter names of published checkpoints."""
import math
import os
import sys

import pytest
import torch
import torch.nn.functional as F

from torchturbo_b200.models.kimi_k25.vision import MoonViT, MoonViTConfig, PatchMergerMLP, init_moonvit

CFG = dict(patch_size=14, init_pos_emb_height=6, init_pos_emb_width=6, init_pos_emb_time=4, vt_num_attention_heads=4,
           vt_num_hidden_layers=2, vt_hidden_size=64, vt_intermediate_size=96, merge_kernel_size=[2, 2], text_hidden_size=48)
GRID = [[1, 6, 6], [1, 4, 8], [3, 2, 4]]            # native grid, resampled grid, a 3-frame clip


def _build(seed=0):
    torch.manual_seed(seed)
    cfg = MoonViTConfig(**CFG)
    tower, proj = MoonViT(cfg, torch.float32), PatchMergerMLP(cfg, torch.float32)
    init_moonvit(tower, proj, 0.05)
    with torch.no_grad():
        for m in list(tower.parameters()) + list(proj.parameters()):
            if m.ndim == 1:
                m.add_(torch.randn_like(m) * 0.1)
    L = sum(t * h * w for t, h, w in GRID)
    pixels = torch.randn(L, 3, 14, 14)
    return cfg, tower, proj, pixels


def _oracle(cfg, sd, psd, pixels, grid):
    C, nh = cfg.vt_hidden_size, cfg.vt_num_attention_heads
    d = C // nh
    x = F.conv2d(pixels, sd["patch_embed.proj.weight"], sd["patch_embed.proj.bias"]).view(pixels.shape[0], -1)
    pw = sd["patch_embed.pos_emb.weight"]
    omega = 1.0 / 10000 ** (torch.arange(C // 2, dtype=torch.float32) / (C / 2.0))
    pos = []
    for t, h, w in grid:
        e = pw.flatten(0, 1) if (h, w) == tuple(pw.shape[:2]) else \
            F.interpolate(pw.permute(2, 0, 1)[None], size=(h, w), mode="bicubic")[0].permute(1, 2, 0).flatten(0, 1)
        if t > 1:
            ang = torch.arange(t, dtype=torch.float32)[:, None] * omega[None]
            e = (e[None] + torch.cat([ang.sin(), ang.cos()], 1)[:, None]).flatten(0, 1)
        pos.append(e)
    x = x + torch.cat(pos)
    # rotary factors as complex numbers: pair 2i <- column, pair 2i+1 <- row
    fr = 1.0 / 10000.0 ** (torch.arange(0, d, 4)[: d // 4].float() / d)
    cis = []
    for t, h, w in grid:
        flat = torch.arange(h * w).float()
        col, row = flat % w, flat // w
        c = torch.cat([torch.polar(torch.ones(h * w, d // 4), torch.outer(col, fr))[..., None],
                       torch.polar(torch.ones(h * w, d // 4), torch.outer(row, fr))[..., None]], -1).reshape(h * w, d // 2)
        cis.append(c.repeat(t, 1))
    cis = torch.cat(cis)[:, None]
    bounds = [0]
    for t, h, w in grid:
        bounds.append(bounds[-1] + t * h * w)
    for i in range(cfg.vt_num_hidden_layers):
        g = lambda n: sd[f"encoder.blocks.{i}.{n}"]  # noqa: E731
        hn = F.layer_norm(x, (C,), g("norm0.weight"), g("norm0.bias"), 1e-5)
        qkv = F.linear(hn, g("wqkv.weight"), g("wqkv.bias")).view(-1, 3, nh, d)
        q, k, v = qkv.unbind(1)
        rot = lambda u: torch.view_as_real(torch.view_as_complex(u.reshape(*u.shape[:-1], -1, 2).contiguous()) * cis).flatten(-2)  # noqa: E731
        q, k = rot(q), rot(k)
        outs = []
        for a, b in zip(bounds[:-1], bounds[1:]):
            s = torch.einsum("qhd,khd->hqk", q[a:b], k[a:b]) / math.sqrt(d)
            outs.append(torch.einsum("hqk,khd->qhd", s.softmax(-1), v[a:b]).reshape(b - a, C))
        x = x + F.linear(torch.cat(outs), g("wo.weight"), g("wo.bias"))
        hn = F.layer_norm(x, (C,), g("norm1.weight"), g("norm1.bias"), 1e-5)
        x = x + F.linear(F.gelu(F.linear(hn, g("mlp.fc0.weight"), g("mlp.fc0.bias")), approximate="tanh"),
                         g("mlp.fc1.weight"), g("mlp.fc1.bias"))
    x = F.layer_norm(x, (C,), sd["encoder.final_layernorm.weight"], sd["encoder.final_layernorm.bias"], 1e-5)
    rows = []
    for (t, h, w), a in zip(grid, bounds[:-1]):
        s = x[a:a + t * h * w].view(t, h // 2, 2, w // 2, 2, C).permute(0, 1, 3, 2, 4, 5).mean(0)
        rows.append(s.reshape(-1, 4, C))
    m = torch.cat(rows)
    m = F.layer_norm(m, (C,), psd["pre_norm.weight"], psd["pre_norm.bias"], cfg.projector_ln_eps).reshape(m.shape[0], -1)
    return F.linear(F.gelu(F.linear(m, psd["proj.0.weight"], psd["proj.0.bias"])), psd["proj.2.weight"], psd["proj.2.bias"])


def test_tower_and_projector_match_the_plain_formulation():
    cfg, tower, proj, pixels = _build()
    with torch.no_grad():
        ours = proj(tower(pixels.reshape(pixels.shape[0], -1), torch.tensor(GRID)))
        ref = _oracle(cfg, tower.state_dict(), proj.state_dict(), pixels, GRID)
    assert ours.shape == ref.shape == (sum(h * w // 4 for _, h, w in GRID), cfg.text_hidden_size)
    assert (ours - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())


def test_parameter_names_are_those_of_published_checkpoints():
    cfg, tower, proj, _ = _build()
    names = set(tower.state_dict()) | {"mm_projector." + k for k in proj.state_dict()}
    want = {"patch_embed.proj.weight", "patch_embed.proj.bias", "patch_embed.pos_emb.weight", "encoder.final_layernorm.weight",
            "encoder.final_layernorm.bias", "mm_projector.pre_norm.weight", "mm_projector.pre_norm.bias",
            "mm_projector.proj.0.weight", "mm_projector.proj.0.bias", "mm_projector.proj.2.weight", "mm_projector.proj.2.bias"}
    for i in range(cfg.vt_num_hidden_layers):
        for n in ("norm0", "norm1", "wqkv", "wo", "mlp.fc0", "mlp.fc1"):
            want |= {f"encoder.blocks.{i}.{n}.weight", f"encoder.blocks.{i}.{n}.bias"}
    assert names == want
    assert tuple(tower.patch_embed.proj.weight.shape) == (64, 3, 14, 14)
    assert tuple(tower.patch_embed.pos_emb.weight.shape) == (6, 6, 64)


def test_gradients_reach_every_parameter():
    cfg, tower, proj, pixels = _build()
    out = proj(tower(pixels.reshape(pixels.shape[0], -1), torch.tensor(GRID)))
    out.square().mean().backward()
    for n, p in list(tower.named_parameters()) + list(proj.named_parameters()):
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, n


def test_against_the_reference_class_when_installed():
    """Same weights through the reference's own MoonViT (needs the offline install of the reference and its
    dependencies; skipped otherwise)."""
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(root, "torchturbo")):
        pytest.skip("reference package not installed")
    sys.path[:0] = [root, os.path.join(os.path.dirname(root), "shims")]
    try:
        try:
            from torchturbo.models.kimi_k25 import modeling_kimi_k25 as R
        except Exception as e:  # noqa: BLE001
            pytest.skip(f"reference modelling code does not import here: {type(e).__name__}")
        cfg, tower, proj, pixels = _build()

        class VC:
            pass

        vc = VC()
        for k, v in CFG.items():
            setattr(vc, k, v)
        vc.pos_emb_type, vc.video_attn_type, vc.merge_type, vc._attn_implementation = "divided_fixed", "spatial_temporal", "sd2_tpool", "eager"
        vc.mm_projector_type, vc.mm_hidden_size, vc.projector_hidden_act, vc.projector_ln_eps = "patchmerger", 64, "gelu", 1e-5
        try:
            rt = R.MoonViT3dPretrainedModel(R.VisionTowerConfig(vc)).float().eval()
            rp = R.PatchMergerMLP(R.ProjectorConfig(vc)).float().eval()
        except Exception as e:  # noqa: BLE001
            pytest.skip(f"reference tower cannot be built on this box: {type(e).__name__}: {e}")
        R.seed_all = lambda *a, **k: None       # the reference reseeds through `torch_npu` in every encoder call
        rt.load_state_dict(tower.state_dict(), strict=True)
        rp.load_state_dict(proj.state_dict(), strict=True)
        # One medium per reference call: its eager attention adds the boolean segment mask to the scores instead of
        # masking with it, so several media in one call attend to each other there (its flash-attention path, which
        # needs a GPU build of flash-attn, separates them by `cu_seqlens` as this tower does).
        with torch.no_grad():
            refs, a = [], 0
            for g in GRID:
                n = g[0] * g[1] * g[2]
                refs += list(rp(rt(pixels[a:a + n], torch.tensor([g]))))
                a += n
            ref = torch.cat(refs)
            ours = proj(tower(pixels.reshape(pixels.shape[0], -1), torch.tensor(GRID)))
        assert (ours - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
    finally:
        del sys.path[:2]
