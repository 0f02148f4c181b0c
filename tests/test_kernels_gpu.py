"""Numerics of every CUDA kernel against a plain PyTorch fp32 formulation of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from torchturbo_b200 import kernels

    assert kernels.available(), "sm_100a library not built"
    return kernels


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert torch.allclose(a, b, rtol=rtol, atol=atol * max(ref, 1e-6)), f"max err {err} (ref max {ref})"


@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (256, 512, 256), (300, 200, 136), (4096, 1536, 2048), (77, 8, 64)])
def test_gemm_nt(K, M, N, K_):
    a, b = _rand(M, K_), _rand(N, K_)
    c = K.gemm(a, b)
    torch.cuda.synchronize()
    assert K.status() == (0, 0)
    _close(c, a.float() @ b.float().t())


@pytest.mark.parametrize("M,N,K_", [(256, 256, 128), (304, 264, 200), (2048, 2048, 768)])
def test_gemm_nn_and_tn(K, M, N, K_):
    a, b = _rand(M, K_), _rand(K_, N)
    _close(K.gemm(a, b, b_mn=True), a.float() @ b.float())
    at = _rand(K_, M)
    _close(K.gemm(at, b, a_mn=True, b_mn=True), at.float().t() @ b.float())
    bk = _rand(N, K_)
    _close(K.gemm(at, bk, a_mn=True, b_mn=False), at.float().t() @ bk.float().t())
    assert K.status() == (0, 0)


def test_gemm_fp32_accumulate_and_residual(K):
    a, b = _rand(512, 256), _rand(384, 256)
    out = torch.ones(512, 384, device="cuda", dtype=torch.float32)
    K.gemm(a, b, out=out, accumulate=True)
    _close(out, a.float() @ b.float().t() + 1.0)
    res = _rand(512, 384)
    c = K.gemm(a, b, residual=res)
    _close(c, a.float() @ b.float().t() + res.float())


def test_gemm_swiglu_epilogue(K):
    M, H, F = 384, 256, 320
    x, w = _rand(M, H), _rand(2 * F, H, scale=0.1)
    scale = torch.rand(M, device="cuda")
    pre = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    y = K.gemm(x, w, swiglu=True, row_scale=scale, preact=pre)
    ref_pre = (x.float() @ w.float().t())
    _close(pre, ref_pre)
    g, u = pre.float()[:, :F], pre.float()[:, F:]
    _close(y, torch.nn.functional.silu(g) * u * scale[:, None])
    # MN-major weights ([H, 2F], the expert layout)
    wt = w.t().contiguous()
    y2 = K.gemm(x, wt, b_mn=True, swiglu=True, row_scale=scale)
    _close(y2, torch.nn.functional.silu(g) * u * scale[:, None])


def test_grouped_gemm(K):
    torch.manual_seed(0)
    E, H, F, T, k = 8, 256, 192, 300, 2
    idx = torch.randint(0, E, (T, k), device="cuda", dtype=torch.int32)
    x = _rand(T, H)
    pm = K.perm_index(idx, E)
    xp, _ = K.perm_scatter(x, pm["row_of"], k, pm["capacity_rows"], counts=pm["counts"], seg_start=pm["seg_start"])
    torch.cuda.synchronize()
    assert int(pm["status"].item()) == 0
    w = _rand(E, H, F, scale=0.1)  # [E, in, out]
    y = K.gemm(xp, w, b_mn=True, tile_group=pm["tile_group"])
    seg = pm["seg_start"].cpu().tolist()
    cnt = pm["counts"].cpu().tolist()
    for e in range(E):
        rows = slice(seg[e], seg[e] + cnt[e])
        _close(y[rows], xp[rows].float() @ w[e].float())
    # dX: grouped with K-major B (w[e] is [H, F] = [N, K] for dX = dY @ w[e]^T)
    dy = _rand(pm["capacity_rows"], F)
    dx = K.gemm(dy, w, b_mn=False, tile_group=pm["tile_group"])
    for e in range(E):
        rows = slice(seg[e], seg[e] + cnt[e])
        _close(dx[rows], dy[rows].float() @ w[e].float().t())
    # dW: grouped-K; pad rows of xp are zero so they add nothing
    dw = K.gemm(xp, dy, a_mn=True, b_mn=True, group_rows=pm["seg_start"], out_dtype=torch.float32)
    for e in range(E):
        rows = slice(seg[e], seg[e + 1])
        _close(dw[e], xp[rows].float().t() @ dy[rows].float())
    assert K.status() == (0, 0)


def test_perm_roundtrip(K):
    torch.manual_seed(1)
    E, H, T, k = 16, 128, 257, 4
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    prob = torch.rand(T, k, device="cuda")
    x = _rand(T, H)
    pm = K.perm_index(idx, E)
    xp, rv = K.perm_scatter(x, pm["row_of"], k, pm["capacity_rows"], counts=pm["counts"], seg_start=pm["seg_start"],
                            val=prob.reshape(-1))
    row_of = pm["row_of"].long()
    # (expert, token) order: rows of one expert are in token order
    flat_e = idx.reshape(-1).long()
    order = torch.argsort(flat_e * (T * k) + torch.arange(T * k, device="cuda"))
    seg = pm["seg_start"].long()
    cnt = torch.bincount(flat_e, minlength=E)
    assert torch.equal(cnt.int(), pm["counts"])
    rank = torch.empty_like(order)
    start_unpadded = torch.cumsum(cnt, 0) - cnt
    rank[order] = torch.arange(T * k, device="cuda") - start_unpadded[flat_e[order]]
    assert torch.equal(row_of, seg[flat_e] + rank)
    assert torch.equal(xp[row_of], x.repeat_interleave(k, 0))
    assert torch.equal(rv[row_of], prob.reshape(-1))
    out = K.perm_combine(xp, pm["row_of"], T, k, weights=prob)
    _close(out, (x.float()[:, None, :] * prob[:, :, None]).sum(1))


def test_rmsnorm(K):
    T, H = 300, 2048
    x, r, w = _rand(T, H), _rand(T, H), _rand(H)
    y, rstd, xs = K.rmsnorm_fwd(x, w, 1e-6, residual=r)
    s = (x.float() + r.float()).bfloat16().float()
    ref = (s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6)).bfloat16().float() * w.float()
    _close(xs, s, atol=1e-2)
    _close(y, ref)
    dy, dres = _rand(T, H), _rand(T, H)
    dx, dw = K.rmsnorm_bwd(dy, xs, w, rstd, dres=dres)
    s_ = s.clone().requires_grad_(True)
    w_ = w.float().clone().requires_grad_(True)
    yy = s_ * torch.rsqrt(s_.pow(2).mean(-1, keepdim=True) + 1e-6) * w_
    yy.backward(dy.float())
    _close(dx, s_.grad + dres.float())
    _close(dw, w_.grad)
    # wide rows
    x2, w2 = _rand(5, 5120), _rand(5120)
    y2, _, _ = K.rmsnorm_fwd(x2, w2, 1e-6)
    _close(y2, (x2.float() * torch.rsqrt(x2.float().pow(2).mean(-1, keepdim=True) + 1e-6)).bfloat16().float() * w2.float())


def test_qknorm_rope(K):
    T, nq, nkv, D = 130, 8, 2, 128
    qkv = _rand(T, (nq + 2 * nkv) * D)
    wq, wk = _rand(D), _rand(D)
    pos = torch.arange(T, device="cuda").float()
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = pos[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    def ref(qkv_f, wq_f, wk_f):
        q = qkv_f[:, : nq * D].reshape(T, nq, D)
        k = qkv_f[:, nq * D: (nq + nkv) * D].reshape(T, nkv, D)

        def nr(x, w):
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
            x1, x2 = x[..., : D // 2], x[..., D // 2:]
            c, s = cos[:, None], sin[:, None]
            return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

        return nr(q, wq_f), nr(k, wk_f)

    q, k, rstd = K.qknorm_rope_fwd(qkv, nq, nkv, D, wq, wk, cos, sin, 1e-6)
    a = qkv.float().requires_grad_(True)
    b, c = wq.float().requires_grad_(True), wk.float().requires_grad_(True)
    qr, kr = ref(a, b, c)
    _close(q, qr)
    _close(k, kr)
    dq, dk = _rand(T, nq, D), _rand(T, nkv, D)
    (qr * dq.float()).sum().add((kr * dk.float()).sum()).backward()
    dqkv = torch.zeros_like(qkv)
    dwq, dwk = K.qknorm_rope_bwd(dq, dk, qkv, nq, nkv, D, wq, wk, cos, sin, rstd, dqkv)
    _close(dqkv[:, : (nq + nkv) * D], a.grad[:, : (nq + nkv) * D])
    _close(dwq, b.grad)
    _close(dwk, c.grad)


def test_swiglu(K):
    R, F = 200, 768
    x = _rand(R, 2 * F)
    sc = torch.rand(R, device="cuda")
    y = K.swiglu_fwd(x, sc)
    xf = x.float().requires_grad_(True)
    s_ = sc.clone().requires_grad_(True)
    ref = torch.nn.functional.silu(xf[:, :F]) * xf[:, F:] * s_[:, None]
    _close(y, ref)
    dy = _rand(R, F)
    ref.backward(dy.float())
    dx, ds = K.swiglu_bwd(dy, x, sc, want_dscale=True)
    _close(dx, xf.grad)
    _close(ds, s_.grad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cross_entropy(K, dtype):
    R, V = 64, 5000
    logits = _rand(R, V, scale=3.0, dtype=dtype)
    labels = torch.randint(0, V, (R,), device="cuda")
    labels[::7] = -100
    grad = torch.empty(R, V, device="cuda", dtype=torch.bfloat16)
    gs = torch.tensor([0.5], device="cuda")
    loss = K.cross_entropy(logits, labels, grad_out=grad, grad_scale=gs)
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels, reduction="none", ignore_index=-100)
    _close(loss, ref, rtol=1e-3, atol=1e-3)
    (ref.sum() * 0.5).backward()
    _close(grad, lf.grad, atol=1e-2)


def test_adamw_and_clip(K):
    torch.manual_seed(0)
    shapes = [(1000,), (70000,), (256, 300)]
    ps = [torch.randn(*s, device="cuda") for s in shapes]
    gs = [torch.randn(*s, device="cuda").bfloat16() if i == 1 else torch.randn(*s, device="cuda") for i, s in enumerate(shapes)]
    ref_p = [p.clone().requires_grad_(True) for p in ps]
    opt = torch.optim.AdamW(ref_p, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
    m = [torch.zeros_like(p) for p in ps]
    v = [torch.zeros_like(p) for p in ps]
    sh = [torch.empty_like(p, dtype=torch.bfloat16) for p in ps]
    plan = K.MultiTensorPlan(ps, m, v, sh)
    for step in (1, 2):
        plan.refresh_grads(gs)
        part = K.grad_sqnorm_partials(plan)
        clip = K.clip_coef(part, 1.0)
        total = math.sqrt(sum(g.float().pow(2).sum().item() for g in gs))
        assert abs(clip[1].item() - total) / total < 1e-4
        K.adamw_step(plan, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step, clip=clip[2:3])
        for rp, g in zip(ref_p, gs):
            rp.grad = g.float() * min(1.0, 1.0 / (total + 1e-6))
        opt.step()
    for p, rp, s in zip(ps, ref_p, sh):
        _close(p, rp.detach(), rtol=1e-4, atol=1e-5)
        _close(s, rp.detach(), atol=1e-2)


def test_fused_adamw_gradient_prescale(K):
    """`FusedAdamW.grad_prescale` (the 1/ep scaling of expert gradients) equals scaling the gradients beforehand,
    in the squared-norm reduction and in the update, and is cleared by `step()`."""
    from torchturbo_b200.engine.optimizers import FusedAdamW

    torch.manual_seed(1)
    a = [torch.randn(300, 70, device="cuda").bfloat16().requires_grad_(True) for _ in range(2)]
    b = [x.detach().clone().requires_grad_(True) for x in a]
    gs = [torch.randn_like(x) for x in a]
    oa, ob = FusedAdamW(a, lr=1e-2), FusedAdamW(b, lr=1e-2)
    for x, y, g in zip(a, b, gs):
        x.grad, y.grad = g.clone(), (g.float() * 0.25).to(g.dtype)
    oa.grad_prescale = 0.25
    sa, sb = oa.grad_sq_sum(), ob.grad_sq_sum()
    _close(sa, sb, rtol=2e-2, atol=1e-3)          # b's gradients were rounded to bf16 after scaling
    oa.step(); ob.step()
    assert oa.grad_prescale == 1.0
    for x, y in zip(a, b):
        _close(x.detach(), y.detach(), atol=2e-2)
        _close(oa.state[x]["master"], ob.state[y]["master"], rtol=2e-2, atol=1e-4)


@pytest.mark.parametrize("score_fn", ["softmax_post", "softmax_pre", "sigmoid"])
def test_router_rows_without_a_finite_logit_select_valid_experts(K, score_fn):
    """A row of NaN (or -inf) logits, e.g. after an upstream exchange gave up, must still select expert ids inside
    [0, E): the ids index histograms and routing tables in later kernels.  The weights of such a row may be NaN."""
    torch.manual_seed(1)
    T, E, k = 64, 128, 8
    logits = torch.randn(T, E, device="cuda")
    logits[3] = float("nan")
    logits[7, ::2] = float("nan")
    logits[11] = float("-inf")
    bias = torch.randn(E, device="cuda")
    out = K.router_fwd(logits, k, score_fn, expert_bias=bias, want_stats=True)
    idx = out["topk_idx"].long()
    assert int(idx.min()) >= 0 and int(idx.max()) < E
    assert int(out["counts"].sum()) == T * k and int(out["aux_counts"].sum()) == T * k
    for t in range(T):
        assert idx[t].unique().numel() == k          # k distinct experts per token
    good = torch.ones(T, dtype=torch.bool, device="cuda")
    good[[3, 7, 11]] = False
    assert torch.isfinite(out["topk_prob"][good]).all()


@pytest.mark.parametrize("score_fn", ["softmax_post", "softmax_pre", "sigmoid"])
def test_router(K, score_fn):
    torch.manual_seed(0)
    T, E, k = 333, 128, 8
    logits = torch.randn(T, E, device="cuda")
    valid = torch.ones(T, dtype=torch.bool, device="cuda")
    valid[-5:] = False
    out = K.router_fwd(logits, k, score_fn, valid_mask=valid, want_stats=True, scaling=2.0)

    def ref(lg):
        if score_fn == "softmax_post":
            tv, ti = torch.topk(lg, k, dim=-1)
            p = torch.softmax(tv, -1)
            sc = torch.softmax(lg, -1)
        elif score_fn == "softmax_pre":
            sc = torch.softmax(lg, -1)
            p, ti = torch.topk(sc, k, dim=-1)
        else:
            s = torch.sigmoid(lg)
            tv, ti = torch.topk(s, k, dim=-1)
            p = tv / (tv.sum(-1, keepdim=True) + 1e-20)
            sc = s / (s.sum(-1, keepdim=True) + 1e-20)
        return p * 2.0, ti, sc

    lg = logits.clone().requires_grad_(True)
    p, ti, sc = ref(lg)
    assert torch.equal(out["topk_idx"].long(), ti)
    _close(out["topk_prob"], p, rtol=1e-4, atol=1e-5)
    _close(out["lse"], torch.logsumexp(logits, -1), rtol=1e-4, atol=1e-5)
    _close(out["score_sum"], (sc * valid[:, None]).sum(0), rtol=1e-3, atol=1e-4)
    cnt = torch.bincount(ti[valid].reshape(-1), minlength=E)
    assert torch.equal(out["aux_counts"].long(), cnt)
    assert torch.equal(out["counts"].long(), torch.bincount(ti.reshape(-1), minlength=E))
    dprob = torch.randn(T, k, device="cuda")
    aux_g = torch.randn(E, device="cuda")
    dlse = (0.02 * out["lse"] * valid).contiguous()
    loss = (p * dprob).sum() + ((sc * valid[:, None]) * aux_g).sum() + 0.01 * (torch.logsumexp(lg, -1)[valid] ** 2).sum()
    loss.backward()
    dl = K.router_bwd(logits, out["topk_idx"], out["topk_prob"], k, score_fn, dprob=dprob, aux_grad=aux_g,
                      lse=out["lse"], valid_mask=valid, dlse=dlse, scaling=2.0)
    _close(dl, lg.grad, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("causal", [True, False])
def test_attention_fwd(K, causal):
    from torchturbo_b200.ops.providers.native import attention_ref

    torch.manual_seed(0)
    T, Hq, Hk, D = 1000, 8, 2, 128
    cu = torch.tensor([0, 130, 131, 600, 900], dtype=torch.int32)  # tokens 900..999 are padding
    qkv = _rand(T, (Hq + 2 * Hk) * D)
    q = qkv[:, : Hq * D].reshape(T, Hq, D).contiguous()
    k = qkv[:, Hq * D: (Hq + Hk) * D].reshape(T, Hk, D).contiguous()
    v = qkv[:, (Hq + Hk) * D:].view(T, Hk, D)  # strided view, as produced by the fused QKV projection
    tiles = K.build_q_tiles(cu).cuda()
    out, lse, ml = K.attn_fwd(q, k, v, tiles, scale=D ** -0.5, causal=causal, want_max_logit=True)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    ref, ref_ml = attention_ref(q, k, v, cu, causal=causal, scale=D ** -0.5, want_max_logits=True)
    _close(out, ref, atol=2e-2)
    _close(ml, ref_ml, rtol=1e-2, atol=1e-2)
    assert float(out[900:].abs().max()) == 0.0
    # lse against a direct computation on one document / head
    a, b = 131, 600
    s = (q[a:b, 3].float() @ k[a:b, 0].float().t()) * D ** -0.5
    if causal:
        s = s.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    _close(lse[3, a:b], torch.logsumexp(s, -1), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("causal", [True, False])
def test_attention_fwd_rescales_in_place_when_a_later_block_raises_the_maximum(K, causal):
    """Keys whose logits grow by far more than 2^8 from one 128-row block to the next (the accumulator in tensor memory is
    rescaled in place) and keys that grow slowly (the running maximum is left stale); output and lse against fp32."""
    from torchturbo_b200.ops.providers.native import attention_ref

    torch.manual_seed(3)
    T, Hq, Hk, D = 900, 4, 2, 128
    cu = torch.tensor([0, 520, 900], dtype=torch.int32)
    q, k, v = (torch.randn(T, Hq if i == 0 else Hk, D, device="cuda") for i in range(3))
    ramp = torch.ones(T, device="cuda")
    ramp[128:256] = 1.5          # a modest rise: no rescale
    ramp[256:384] = 9.0          # far beyond the threshold
    ramp[384:520] = 0.2
    ramp[520 + 300:] = 7.0
    q, k, v = q.bfloat16(), (k * ramp[:, None, None]).bfloat16(), v.bfloat16()
    tiles = K.build_q_tiles(cu).cuda()
    out, lse, ml = K.attn_fwd(q, k, v, tiles, scale=D ** -0.5, causal=causal, want_max_logit=True)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    ref, ref_ml = attention_ref(q, k, v, cu, causal=causal, scale=D ** -0.5, want_max_logits=True)
    _close(out, ref, atol=3e-2)
    _close(ml, ref_ml, rtol=1e-2, atol=1e-2)
    for a, b, hq in ((0, 520, 1), (520, 900, 2)):
        sc = (q[a:b, hq].float() @ k[a:b, hq // 2].float().t()) * D ** -0.5
        if causal:
            sc = sc.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool, device="cuda").tril(), float("-inf"))
        _close(lse[hq, a:b], torch.logsumexp(sc, -1), rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("causal", [True, False])
def test_attention_bwd(K, causal):
    from torchturbo_b200.ops.providers.native import attention_ref

    torch.manual_seed(1)
    T, Hq, Hk, D = 700, 4, 2, 128
    cu = torch.tensor([0, 200, 201, 520, 650], dtype=torch.int32)
    q, k, v = _rand(T, Hq, D), _rand(T, Hk, D), _rand(T, Hk, D)
    tiles = K.build_q_tiles(cu).cuda()
    out, lse, _ = K.attn_fwd(q, k, v, tiles, scale=D ** -0.5, causal=causal)
    dout = _rand(T, Hq, D)
    dq, dk, dv = K.attn_bwd(dout, q, k, v, out, lse, tiles, scale=D ** -0.5, causal=causal)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, cu, causal=causal, scale=D ** -0.5)
    ref.backward(dout.float())
    _close(dq, qf.grad, atol=3e-2)
    _close(dk, kf.grad, atol=3e-2)
    _close(dv, vf.grad, atol=3e-2)
    assert float(dk[650:].abs().max()) == 0.0 and float(dq[650:].abs().max()) == 0.0


@pytest.mark.parametrize("causal", [True, False])
def test_latent_attention_widths_forward_and_backward(K, causal):
    """Query / key heads 192 wide with 128-wide values (multi-head latent attention): forward, dK / dV from the
    kv-major kernel and dQ from the query-major pass, against the fp32 formulation."""
    from torchturbo_b200.ops.providers.native import attention_ref

    torch.manual_seed(4)
    T, H, Dqk, Dv = 700, 4, 192, 128
    cu = torch.tensor([0, 200, 201, 520, 650], dtype=torch.int32)
    q, k, v = _rand(T, H, Dqk), _rand(T, H, Dqk), _rand(T, H, Dv)
    tiles, kv_tiles = K.build_q_tiles(cu).cuda(), K.build_kv_tiles(cu).cuda()
    scale = Dqk ** -0.5
    out, lse, ml = K.attn_fwd(q, k, v, tiles, scale=scale, causal=causal, want_max_logit=True)
    assert out.shape == (T, H, Dv)
    dout = _rand(T, H, Dv)
    dq, dk, dv = K.attn_bwd(dout, q, k, v, out, lse, kv_tiles, scale=scale, causal=causal, q_tiles_dev=tiles)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref, ref_ml = attention_ref(qf, kf, vf, cu, causal=causal, scale=scale, want_max_logits=True)
    ref.backward(dout.float())
    _close(out, ref, atol=2e-2)
    _close(ml, ref_ml, rtol=1e-2, atol=1e-2)
    _close(dq, qf.grad, atol=3e-2)
    _close(dk, kf.grad, atol=3e-2)
    _close(dv, vf.grad, atol=3e-2)
    assert float(out[650:].abs().max()) == 0.0 and float(dq[650:].abs().max()) == 0.0 and float(dk[650:].abs().max()) == 0.0


def test_deterministic_attention_backward_is_bit_reproducible_and_matches_the_default(K):
    from torchturbo_b200.ops.providers.native import attention_ref

    torch.manual_seed(5)
    T, Hq, Hk, D = 900, 4, 4, 128
    cu = torch.tensor([0, 300, 900], dtype=torch.int32)
    q, k, v = _rand(T, Hq, D), _rand(T, Hk, D), _rand(T, Hk, D)
    tiles, kv_tiles = K.build_q_tiles(cu).cuda(), K.build_kv_tiles(cu).cuda()
    out, lse, _ = K.attn_fwd(q, k, v, tiles, scale=D ** -0.5, causal=True)
    dout = _rand(T, Hq, D)
    runs = [K.attn_bwd(dout, q, k, v, out, lse, kv_tiles, scale=D ** -0.5, causal=True, q_tiles_dev=tiles, deterministic=True)
            for _ in range(3)]
    fast = K.attn_bwd(dout, q, k, v, out, lse, kv_tiles, scale=D ** -0.5, causal=True)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    for r in runs[1:]:
        assert all(torch.equal(a, b) for a, b in zip(r, runs[0]))
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    attention_ref(qf, kf, vf, cu, causal=True, scale=D ** -0.5).backward(dout.float())
    for got, fast_g, want in zip(runs[0], fast, (qf.grad, kf.grad, vf.grad)):
        _close(got, want, atol=3e-2)
        _close(got, fast_g.float(), atol=3e-2)
    # grouped-query heads (one CTA per kv head walks its four query heads): bit-reproducible too, through the operator
    # with the global switch on
    from torchturbo_b200.ops.providers import b200_attention as BA

    q2, k2, v2 = _rand(T, 8, D), _rand(T, 2, D), _rand(T, 2, D)
    g2 = _rand(T, 8, D)
    grads = []
    torch.use_deterministic_algorithms(True)
    try:
        for _ in range(3):
            leaves = [t.clone().requires_grad_(True) for t in (q2, k2, v2)]
            BA.B200Attention()(*leaves, cu, 600, causal=True, scale=D ** -0.5).backward(g2)
            grads.append([t.grad for t in leaves])
    finally:
        torch.use_deterministic_algorithms(False)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    for r in grads[1:]:
        assert all(torch.equal(a, b) for a, b in zip(r, grads[0]))
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q2, k2, v2))
    attention_ref(qf, kf, vf, cu, causal=True, scale=D ** -0.5).backward(g2.float())
    for got, want in zip(grads[0], (qf.grad, kf.grad, vf.grad)):
        _close(got, want, atol=3e-2)


def test_narrow_heads_run_on_the_tcgen05_kernel_with_zero_padding(K):
    """ViT-style attention (head width 72, full attention, no GQA) through the operator: zero-padded to 128 columns on
    the library's own kernel, forward and backward against the fp32 formulation."""
    from torchturbo_b200.ops.providers import b200_attention as BA
    from torchturbo_b200.ops.providers.native import attention_ref

    torch.manual_seed(2)
    T, H, D = 500, 4, 72
    cu = torch.tensor([0, 196, 452, 500], dtype=torch.int32)
    q, k, v = (_rand(T, H, D).requires_grad_(True) for _ in range(3))
    before = K.launch_count()
    out = BA.B200Attention()(q, k, v, cu, 256, causal=False, scale=D ** -0.5)
    assert K.launch_count() > before and out.shape == (T, H, D)
    g = _rand(T, H, D)
    out.backward(g)
    torch.cuda.synchronize()
    assert K.attn_status() == (0, 0)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, cu, causal=False, scale=D ** -0.5)
    ref.backward(g.float())
    _close(out, ref, atol=2e-2)
    _close(q.grad, qf.grad, atol=3e-2); _close(k.grad, kf.grad, atol=3e-2); _close(v.grad, vf.grad, atol=3e-2)
    o2, ml = BA.B200AttentionWithMaxLogits()(q.detach(), k.detach(), v.detach(), cu, 256, causal=False, scale=D ** -0.5)
    _, ref_ml = attention_ref(qf, kf, vf, cu, causal=False, scale=D ** -0.5, want_max_logits=True)
    _close(ml, ref_ml, rtol=1e-2, atol=1e-2)


def test_adamw_swap_pipelined_matches_torch(K):
    """Host-resident AdamW state streamed through a two-slot device workspace (chunks smaller than the parameters)."""
    from torchturbo_b200.engine.optimizers import AdamWSwap

    torch.manual_seed(0)
    a = [torch.nn.Parameter(torch.randn(300, 70, device="cuda")), torch.nn.Parameter(torch.randn(5000, device="cuda"))]
    b = [torch.nn.Parameter(p.detach().clone()) for p in a]
    oa = AdamWSwap(a, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95), chunk_elems=4096)
    ob = torch.optim.AdamW(b, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    for _ in range(3):
        for pa, pb in zip(a, b):
            g = torch.randn_like(pa)
            pa.grad, pb.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    assert max((pa - pb).abs().max().item() for pa, pb in zip(a, b)) < 1e-5
    st = oa.state[a[0]]
    assert st["exp_avg"].device.type == "cpu" and st["exp_avg"].is_pinned()
    assert torch.allclose(st["master"].view_as(a[0]).cuda(), a[0].detach(), atol=0)


def test_ulysses_peer_kernels_single_rank(K, tmp_path):
    """The peer-memory Ulysses kernels on a one-rank group (the peer is this GPU): fused QK-norm + RoPE + head scatter
    against the separate QK-norm + RoPE kernel, and the gather / scatter round trip with gradients."""
    import torch.distributed as dist

    from torchturbo_b200.comm import ulysses_p2p

    created = False
    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method=f"file://{tmp_path}/rdzv", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
        created = True
    try:
        Tl, nq, nkv, D = 200, 8, 2, 128
        qkv = _rand(Tl, (nq + 2 * nkv) * D).requires_grad_(True)
        wq, wk = (_rand(D) * 0.1 + 1.0).requires_grad_(True), (_rand(D) * 0.1 + 1.0).requires_grad_(True)
        pos = torch.arange(Tl, device="cuda").float()
        inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
        cos, sin = (pos[:, None] * inv[None]).cos().contiguous(), (pos[:, None] * inv[None]).sin().contiguous()
        q, k, v, ws = ulysses_p2p.qkv_exchange(qkv, nq, nkv, wq, wk, cos, sin, 1e-6, dist.group.WORLD)
        q_ref, k_ref, _ = K.qknorm_rope_fwd(qkv.detach(), nq, nkv, D, wq.detach(), wk.detach(), cos, sin, 1e-6, True)
        _close(q, q_ref, rtol=1e-2, atol=1e-2)          # same formula; fused multiply-adds may round differently
        _close(k, k_ref, rtol=1e-2, atol=1e-2)
        assert torch.equal(v, qkv.detach()[:, (nq + nkv) * D:].view(Tl, nkv, D))
        out = ulysses_p2p.out_exchange(q * 1.0, ws)
        assert torch.equal(out, q)
        g = _rand(Tl, nq, D)
        (out.float() * g.float()).sum().backward()
        torch.cuda.synchronize()
        ws.check()
        # reference gradient through the separate kernels
        dqkv = torch.empty_like(qkv)
        dqkv[:, (nq + nkv) * D:] = 0
        rstd = K.qknorm_rope_fwd(qkv.detach(), nq, nkv, D, wq.detach(), wk.detach(), cos, sin, 1e-6, True)[2]
        dwq, dwk = K.qknorm_rope_bwd(g.contiguous(), torch.zeros(Tl, nkv, D, device="cuda", dtype=torch.bfloat16), qkv.detach(),
                                     nq, nkv, D, wq.detach(), wk.detach(), cos, sin, rstd, dqkv, True)
        _close(qkv.grad[:, : nq * D], dqkv[:, : nq * D])
        _close(wq.grad, dwq)
        assert float(qkv.grad[:, nq * D:].abs().max()) == 0.0
    finally:
        if created:
            dist.destroy_process_group()


def test_newton_schulz_on_tcgen05_gemm(K):
    """Muon's orthogonalisation through the library GEMM against the torch bmm formulation."""
    from torchturbo_b200.engine.optimizers import muon

    torch.manual_seed(0)
    G = torch.randn(3, 256, 512, device="cuda")
    coeffs = (3.4445, -4.7750, 2.0315)
    got = muon.newton_schulz(G, 5, coeffs, 1e-7)
    X = G.to(torch.bfloat16)
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True) + 1e-7).to(X.dtype)
    for _ in range(5):
        A = X @ X.transpose(-2, -1)
        B = torch.baddbmm(A, A, A, beta=coeffs[1], alpha=coeffs[2])
        X = torch.baddbmm(X, B, X, beta=coeffs[0], alpha=1.0)
    assert got.shape == G.shape
    _close(got, X, rtol=5e-2, atol=5e-2)
    s = torch.linalg.svdvals(got[0].float())
    assert float(s.max()) < 1.3 and float(s.min()) > 0.3          # singular values pulled towards one


def _single_rank_group(tmp_path):
    import torch.distributed as dist

    if dist.is_initialized():
        return False
    dist.init_process_group("nccl", init_method=f"file://{tmp_path}/rdzv", rank=0, world_size=1,
                            device_id=torch.device("cuda", torch.cuda.current_device()))
    return True


def test_bounded_peer_wait_gives_up_and_reports(K, tmp_path):
    """A wait on a flag that nothing sets ends after its time budget, records {site, peer} in the status word and
    leaves the context usable (the failure path of every peer-memory kernel; nothing here traps or spins forever)."""
    import time

    import torch.distributed as dist

    from torchturbo_b200.comm.symm import SymmetricBuffer

    created = _single_rank_group(tmp_path)
    try:
        buf = SymmetricBuffer(4096, dist.group.WORLD)
        ch = buf.channel()
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        K.comm_status(reset=True)
        t0 = time.time()
        K.flag_wait(buf.peer_ptrs, ch.offset, 0, 1, ch.next(), 20, status)      # 20 ms budget, flag stays 0
        torch.cuda.synchronize()
        assert time.time() - t0 < 5.0
        code = int(status.item())
        assert code & 0x10000 and (code >> 8) & 0xFF == 2 and code & 0xFF == 0, hex(code)   # site 2 (flag_wait), peer 0
        first, n = K.comm_status(reset=True)
        assert n >= 1 and first != 0
        # once a workspace has failed, later waits return at once instead of stalling for another budget
        t0 = time.time()
        K.flag_wait(buf.peer_ptrs, ch.offset, 0, 1, ch.next(), 2000, status)
        torch.cuda.synchronize()
        assert time.time() - t0 < 1.0
        K.comm_status(reset=True)
        # a satisfied wait is silent, and the GPU still computes
        status.zero_()
        e = ch.next()
        K.flag_signal(buf.peer_ptrs, ch.offset, 0, 1, e)
        K.flag_wait(buf.peer_ptrs, ch.offset, 0, 1, e, 20, status)
        a, b = _rand(128, 64), _rand(128, 64)
        _close(K.gemm(a, b), a.float() @ b.float().t())
        assert int(status.item()) == 0 and K.comm_status() == (0, 0)
    finally:
        if created:
            dist.destroy_process_group()


def test_ep_exchange_writes_every_row_once_and_is_deterministic(K, tmp_path):
    """Expert-parallel dispatch / combine kernels on a one-rank group with poisoned buffers: every routed row lands
    exactly once in its expert's segment, padding rows are zero, nothing else is touched, and two runs agree bitwise."""
    import torch.distributed as dist

    from torchturbo_b200.comm import ep_p2p

    created = _single_rank_group(tmp_path)
    try:
        T, H, E, k = 300, 64, 8, 2
        torch.manual_seed(3)
        x = _rand(T, H)
        idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
        prob = torch.rand(T, k, device="cuda")
        ws = ep_p2p.EPWorkspace(dist.group.WORLD, H, E, T, k, 2.0)
        counts = torch.zeros(E, dtype=torch.int32, device="cuda")
        counts.scatter_add_(0, idx.reshape(-1).long(), torch.ones(T * k, dtype=torch.int32, device="cuda"))
        outs = []
        for _ in range(2):
            ws.recv_rows.fill_(float("nan"))
            ws.recv_vals.fill_(float("nan"))
            xp, rp, seg_start, recv_counts, tile_group, dest_row, expert = ep_p2p._Dispatch.apply(x, prob, idx, counts, ws)
            torch.cuda.synchronize()
            ws.check()
            assert torch.equal(recv_counts, counts)
            seg = seg_start.tolist()
            dr = dest_row.view(T, k)
            assert dr.unique().numel() == T * k                      # no two (token, slot) pairs share a row
            for e in range(E):
                n = int(counts[e])
                rows = xp[seg[e]:seg[e] + n]
                toks = (idx == e).nonzero()[:, 0]
                inside = dr[idx == e]
                assert int(inside.min()) >= seg[e] and int(inside.max()) < seg[e] + n if n else True
                assert not torch.isnan(rows).any()
                assert torch.equal(xp[dr[idx == e].long()], x[toks])          # each row is its token, bit for bit
                pad = xp[seg[e] + n:seg[e + 1]]
                assert float(pad.abs().max()) == 0.0 if pad.numel() else True # padding zeroed, not poison
            used = torch.zeros(xp.shape[0], dtype=torch.bool, device="cuda")
            for e in range(E):
                used[seg[e]:seg[e + 1]] = True
            assert torch.isnan(xp[~used]).all()                      # rows outside every segment were never written
            y = ep_p2p._Combine.apply(xp.clone(), expert, dest_row, seg_start, recv_counts, ws, T, k, None)
            torch.cuda.synchronize()
            _close(y, x.float() * k, rtol=1e-2, atol=1e-2)           # identity experts: k copies of the token
            outs.append((xp.clone(), y.clone(), dest_row.clone()))
        assert torch.equal(outs[0][1], outs[1][1])                   # run-twice determinism of the combined output
        assert torch.equal(outs[0][0].nan_to_num(), outs[1][0].nan_to_num()) and torch.equal(outs[0][2], outs[1][2])
    finally:
        if created:
            dist.destroy_process_group()


@pytest.mark.parametrize("H", [1152, 4304, 64])
def test_layernorm(K, H):
    import torch.nn.functional as F

    torch.manual_seed(0)
    T = 333
    x = (_rand(T, H) * 2 + 0.5).requires_grad_(True)
    w, b = (_rand(H) * 0.1 + 1.0).requires_grad_(True), (_rand(H) * 0.1).requires_grad_(True)
    y, mean, rstd = K.layernorm_fwd(x.detach(), w.detach(), b.detach(), 1e-6)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    ref = F.layer_norm(xf, (H,), wf, bf, 1e-6)
    _close(y, ref, atol=1e-2)
    _close(mean, xf.mean(-1), rtol=1e-3, atol=1e-3)
    dy = _rand(T, H)
    dx, dw, db = K.layernorm_bwd(dy, x.detach(), w.detach(), mean, rstd)
    ref.backward(dy.float())
    _close(dx, xf.grad, atol=2e-2)
    _close(dw, wf.grad, rtol=2e-2, atol=1e-2)
    _close(db, bf.grad, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("act", [None, "gelu_tanh", "gelu"])
@pytest.mark.parametrize("with_res", [False, True])
def test_bias_act(K, act, with_res):
    from torchturbo_b200.ops.providers.native import bias_act_ref

    torch.manual_seed(1)
    R, Cn = 777, 4304
    x, bias = _rand(R, Cn), _rand(Cn)
    res = _rand(R, Cn) if with_res else None
    y = K.bias_act_fwd(x, bias, act, res)
    xf, bf = x.float().requires_grad_(True), bias.float().requires_grad_(True)
    rf = res.float().requires_grad_(True) if with_res else None
    ref = bias_act_ref(xf, bf, act, rf)
    _close(y, ref, atol=1e-2)
    dy = _rand(R, Cn)
    dx, db = K.bias_act_bwd(dy, x, bias, act)
    ref.backward(dy.float())
    _close(dx, xf.grad, atol=2e-2)
    _close(db, bf.grad, rtol=2e-2, atol=2e-2)
    if act is None:
        assert dx.data_ptr() == dy.data_ptr()


def test_vision_block_kernel_path_matches_torch_path(K):
    """One ViT block (LayerNorm, biased projections, full attention at head width 72, GELU MLP) on the kernels
    against the same module evaluated with the torch operator implementations in fp32."""
    from torchturbo_b200.models.qwen3_vl.modeling import Qwen3VLVisionConfig, VisionBlock

    torch.manual_seed(0)
    cfg = Qwen3VLVisionConfig(hidden_size=1152, num_heads=16, intermediate_size=4304)
    blk = VisionBlock(cfg, dtype=torch.bfloat16).cuda()
    P = 320
    cu = torch.tensor([0, 64, 320], dtype=torch.int32)
    x = _rand(P, 1152).requires_grad_(True)
    pos = torch.arange(P, device="cuda").float()
    inv = 1.0 / (10000 ** (torch.arange(0, 36, device="cuda").float() / 36))
    ang = pos[:, None] * inv[None]
    cos, sin = ang.cos(), ang.sin()
    before = K.launch_count()
    y = blk(x, cos, sin, cu, 256)
    assert K.launch_count() - before >= 11      # 2 norms, 4 GEMMs, 4 bias/act tails, attention
    g = _rand(P, 1152)
    y.backward(g)
    ref_blk = VisionBlock(cfg, dtype=torch.float32).cuda()
    ref_blk.load_state_dict({k: v.float() for k, v in blk.state_dict().items()})
    xr = x.detach().float().requires_grad_(True)
    yr = ref_blk(xr, cos, sin, cu, 256)          # fp32 operands: every operator takes its torch formulation
    yr.backward(g.float())
    _close(y, yr, atol=3e-2)
    _close(x.grad, xr.grad, atol=5e-2)
    _close(blk.mlp.linear_fc1.bias.grad, ref_blk.mlp.linear_fc1.bias.grad, rtol=5e-2, atol=5e-2)
    _close(blk.norm1.weight.grad, ref_blk.norm1.weight.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("W,silu,with_bias", [(4, True, False), (4, False, True), (7, True, True), (2, True, False)])
def test_causal_conv1d(K, W, silu, with_bias):
    """Depthwise causal short convolution over a packed row (no leakage across sequence starts), forward and
    backward, against the torch formulation in fp32; also through the operator (autograd)."""
    from torchturbo_b200.ops.providers import b200 as B
    from torchturbo_b200.ops.providers.native_linear_attention import causal_conv1d_ref

    torch.manual_seed(W)
    T, D = 900, 1024 + 64
    cu = torch.tensor([0, 1, 300, 303, 820], dtype=torch.int32)       # sequences of length 1 and 3; tokens 820.. are padding
    x = _rand(1, T, D).requires_grad_(True)
    w = (_rand(D, W) * 0.5).requires_grad_(True)
    b = (_rand(D) * 0.1).requires_grad_(True) if with_bias else None
    act = "silu" if silu else None
    y, _ = B.B200CausalConv1d()(x, w, b, activation=act, cu_seqlens=cu)
    cu_full = torch.cat((cu, torch.tensor([T], dtype=torch.int32)))
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    bf = b.detach().float().requires_grad_(True) if with_bias else None
    ref, _ = causal_conv1d_ref(xf, wf, bf, act, None, False, cu_full)
    _close(y, ref, atol=2e-2)
    g = _rand(1, T, D)
    y.backward(g)
    ref.backward(g.float())
    _close(x.grad, xf.grad, atol=3e-2)
    _close(w.grad, wf.grad, rtol=3e-2, atol=3e-2)
    if with_bias:
        _close(b.grad, bf.grad, rtol=3e-2, atol=3e-2)


def test_ep_exchange_tables_for_eight_ranks_emulated(K, tmp_path):
    """The count-exchange kernel as rank r of an 8-rank group on one GPU: the other ranks' counts and flags are put
    in place by the host (all eight "peer" buffers are this GPU's buffer, so nothing waits), and the tables the kernel
    derives from the 8 x 128 matrix are compared with a direct computation."""
    import ctypes as C

    import torch.distributed as dist

    from torchturbo_b200.comm.symm import SymmetricBuffer

    created = _single_rank_group(tmp_path)
    try:
        W, E = 8, 128
        El = E // W
        g = torch.Generator().manual_seed(5)
        mat = torch.randint(0, 700, (W, E), generator=g, dtype=torch.int32)
        mat[3, 17] = 0
        mat[:, 40] = 0                                              # an expert nobody routes to
        buf = SymmetricBuffer(4 * W * E + 4 * W + 1024, dist.group.WORLD)
        off_counts, counts_all = buf.carve(4 * W * E, torch.int32)
        off_flags, flags = buf.carve(4 * W, torch.int32)
        ptrs = (C.c_ulonglong * W)(*([buf.peer_ptrs[0]] * W))
        for rank in (0, 5, 7):
            counts_all.copy_(mat.reshape(-1))
            counts_all.view(W, E)[rank].zero_()                     # the kernel itself publishes this rank's row
            flags.fill_(1)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            cap_tiles = 4096
            seg_start, recv_counts, tile_group, dest_base = K.ep_exchange(ptrs, off_counts, off_flags, mat[rank].cuda(), rank, W, E,
                                                                          1, 50, cap_tiles, status)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            assert torch.equal(counts_all.view(W, E).cpu(), mat)
            tot = mat.sum(0)                                        # rows every expert receives
            aligned = (tot + 127) // 128 * 128
            for o in range(W):
                seg_o = torch.cat((torch.zeros(1, dtype=torch.int64), aligned[o * El:(o + 1) * El].cumsum(0)))
                before = mat[:rank, o * El:(o + 1) * El].sum(0)
                assert torch.equal(dest_base[o * El:(o + 1) * El].cpu().long(), seg_o[:-1] + before), (rank, o)
                if o == rank:
                    assert torch.equal(seg_start.cpu().long(), seg_o)
                    assert torch.equal(recv_counts.cpu(), tot[o * El:(o + 1) * El].to(torch.int32))
                    tg = tile_group.cpu()
                    for m in range(int(seg_o[-1]) // 128 + 2):
                        row = m * 128
                        want = -1
                        if row < int(seg_o[-1]):
                            want = int((seg_o[1:] > row).nonzero()[0])
                        assert int(tg[m]) == want, (rank, m)
        assert K.comm_status() == (0, 0)
    finally:
        if created:
            dist.destroy_process_group()


def test_fused_aux_loss_matches_the_torch_chain(K):
    from torchturbo_b200.models.modules.moe.moe import _FusedAuxLoss

    torch.manual_seed(0)
    E, k, coeff = 128, 8, 1e-3
    score = torch.rand(E, device="cuda").requires_grad_(True)
    cnt = torch.randint(0, 400, (E,), device="cuda", dtype=torch.int32)
    aux, unscaled = _FusedAuxLoss.apply(score, cnt, k, float(E * coeff), coeff)
    (aux * 3.0).backward()
    s2 = score.detach().clone().requires_grad_(True)
    tpe = cnt.float()
    n = (tpe.sum() / k).clamp(min=1.0)
    ref = (s2 * tpe).sum() * (E * coeff) / (k * n * n)
    (ref * 3.0).backward()
    assert torch.allclose(aux, ref, rtol=1e-5, atol=1e-8) and torch.allclose(unscaled, ref / coeff, rtol=1e-5)
    assert torch.allclose(score.grad, s2.grad, rtol=1e-5, atol=1e-10)
    z, _ = _FusedAuxLoss.apply(score.detach(), torch.zeros_like(cnt), k, float(E * coeff), coeff)
    assert float(z) == 0.0


def test_latent_attention_mixer_runs_on_the_tcgen05_kernels(K):
    """The multi-head latent attention mixer (192-wide query / key heads, 128-wide values) in bf16 on CUDA against the
    same module in fp32 on the CPU; the attention goes to this library's kernels, not to the flash-attn fallback."""
    from types import SimpleNamespace

    from torchturbo_b200.models.modules.mixers import MixerContext, MLAttention
    from torchturbo_b200.ops.providers import b200_attention as BA

    cfg = SimpleNamespace(hidden_size=256, num_attention_heads=4, q_lora_rank=64, kv_lora_rank=64, qk_nope_head_dim=128,
                          qk_rope_head_dim=64, v_head_dim=128, rms_norm_eps=1e-6, rope_interleave=True)
    torch.manual_seed(0)
    ref = MLAttention(cfg, 0).float()
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    dev = MLAttention(cfg, 0).float()
    dev.load_state_dict(ref.state_dict())
    dev = dev.cuda().bfloat16()
    T = 300
    x = (torch.randn(T, 256) * 0.5).bfloat16()
    cu = torch.tensor([0, 130, 300], dtype=torch.int32)
    pos = torch.cat((torch.arange(130), torch.arange(170))).float()
    ang = pos[:, None] * (10000.0 ** (-torch.arange(32).float() / 32))[None]
    ctx_c = MixerContext(cos=ang.cos(), sin=ang.sin(), cu_seqlens=cu, max_seqlen=170)
    ctx_g = MixerContext(cos=ang.cos().cuda(), sin=ang.sin().cuda(), cu_seqlens=cu, max_seqlen=170)
    xc = x.float().requires_grad_(True)
    want = ref(xc, ctx_c)
    g = torch.randn_like(want)
    want.backward(g)
    fallback = []
    orig = BA._LIB_FALLBACK
    BA._LIB_FALLBACK = lambda *a, **kw: fallback.append(1) or orig(*a, **kw)
    try:
        xg = x.cuda().requires_grad_(True)
        got = dev(xg, ctx_g)
        got.backward(g.cuda().bfloat16())
    finally:
        BA._LIB_FALLBACK = orig
    torch.cuda.synchronize()
    assert not fallback and K.attn_status() == (0, 0)
    _close(got.cpu(), want, atol=3e-2)
    _close(xg.grad.cpu(), xc.grad, atol=5e-2)
    for (n, a), b in zip(dev.named_parameters(), ref.parameters()):
        assert (a.grad.float().cpu() - b.grad).abs().max() <= 5e-2 * max(1.0, float(b.grad.abs().max())), n
