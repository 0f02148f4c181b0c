"""Device-timed microbenchmarks of the sm_100a kernels with roofline fractions.

    python -m torchturbo_b200.benchmarks.kernel_bench [gemm] [grouped] [elementwise] [attention] [delta]

Timing rules: 3+ warm-up launches, CUDA events on the launching stream, an L2 flush (write of a
256 MiB buffer) between timed launches, best and median of the timed launches reported.  The
denominators come from MEASURED_PEAKS.json at the repository root when present (cuBLAS bf16
throughput and copy bandwidth measured on the same pool), else from the documented fallback.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

from .. import kernels as K


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"tflops": d["bf16_tflops"], "gbs": d["hbm_gbs"], "src": "measured"}
    return {"tflops": 1590.0, "gbs": 6650.0, "src": "fallback"}


_flush = None


def time_fn(fn, iters=10, warmup=3, flush=True):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[0], ts[len(ts) // 2]


def bench_gemm():
    pk = peaks()
    rows = []
    shapes = [
        (8192, 8192, 8192), (4096, 5120, 2048), (4096, 2048, 4096), (8192, 6144, 4096), (8192, 4096, 4096),
        (8192, 24576, 4096), (8192, 4096, 12288), (4096, 151936, 2048),
    ]
    for M, N, Kd in shapes:
        a = torch.randn(M, Kd, device="cuda").bfloat16()
        b = torch.randn(N, Kd, device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * Kd
        t_ours, m_ours = time_fn(lambda: K.gemm(a, b, out=out))
        t_ref, m_ref = time_fn(lambda: torch.matmul(a, b.t(), out=out))
        rows.append(dict(op="gemm_nt", M=M, N=N, K=Kd, ours_ms=t_ours, ours_med_ms=m_ours, cublas_ms=t_ref,
                         ours_tflops=fl / t_ours / 1e9, cublas_tflops=fl / t_ref / 1e9,
                         frac_of_peak=fl / t_ours / 1e9 / pk["tflops"], peak_src=pk["src"]))
        print(json.dumps(rows[-1]), flush=True)
    # backward orientations on one shape
    M, N, Kd = 8192, 4096, 4096
    a = torch.randn(M, Kd, device="cuda").bfloat16()
    bkn = torch.randn(Kd, N, device="cuda").bfloat16()
    akm = torch.randn(Kd, M, device="cuda").bfloat16()
    fl = 2.0 * M * N * Kd
    for name, fn, ref in [
        ("gemm_nn", lambda: K.gemm(a, bkn, b_mn=True), lambda: a @ bkn),
        ("gemm_tn", lambda: K.gemm(akm, bkn, a_mn=True, b_mn=True), lambda: akm.t() @ bkn),
    ]:
        t_ours, _ = time_fn(fn)
        t_ref, _ = time_fn(ref)
        rows.append(dict(op=name, M=M, N=N, K=Kd, ours_ms=t_ours, cublas_ms=t_ref, ours_tflops=fl / t_ours / 1e9,
                         cublas_tflops=fl / t_ref / 1e9, frac_of_peak=fl / t_ours / 1e9 / pk["tflops"]))
        print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_grouped():
    pk = peaks()
    rows = []
    for E, T, k, H, F in [(16, 32768, 1, 2048, 768), (128, 4096, 8, 2048, 768)]:
        idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32) if k > 1 else \
            torch.randint(0, E, (T, 1), device="cuda", dtype=torch.int32)
        x = torch.randn(T, H, device="cuda").bfloat16()
        pm = K.perm_index(idx, E)
        xp, rv = K.perm_scatter(x, pm["row_of"], k, pm["capacity_rows"], counts=pm["counts"],
                                seg_start=pm["seg_start"], val=torch.rand(T * k, device="cuda"))
        w1 = (torch.randn(E, H, 2 * F, device="cuda") * 0.02).bfloat16()
        w2 = (torch.randn(E, F, H, device="cuda") * 0.02).bfloat16()
        R = T * k
        pre = torch.empty(pm["capacity_rows"], 2 * F, device="cuda", dtype=torch.bfloat16)
        t1, _ = time_fn(lambda: K.gemm(xp, w1, b_mn=True, tile_group=pm["tile_group"], swiglu=True, row_scale=rv, preact=pre))
        act = K.gemm(xp, w1, b_mn=True, tile_group=pm["tile_group"], swiglu=True, row_scale=rv)
        t2, _ = time_fn(lambda: K.gemm(act, w2, b_mn=True, tile_group=pm["tile_group"]))
        dy = torch.randn(pm["capacity_rows"], 2 * F, device="cuda").bfloat16()
        t3, _ = time_fn(lambda: K.gemm(xp, dy, a_mn=True, b_mn=True, group_rows=pm["seg_start"], out_dtype=torch.float32))
        t4, _ = time_fn(lambda: K.gemm(dy, w1, b_mn=False, tile_group=pm["tile_group"]))
        t5, _ = time_fn(lambda: K.gemm(xp, dy, a_mn=True, b_mn=True, group_rows=pm["seg_start"]))
        for name, t, fl in [("fc1_swiglu", t1, 2.0 * R * H * 2 * F), ("fc2", t2, 2.0 * R * F * H),
                            ("dW1", t3, 2.0 * R * H * 2 * F), ("dX1", t4, 2.0 * R * H * 2 * F),
                            ("dW1_bf16_out", t5, 2.0 * R * H * 2 * F)]:
            rows.append(dict(op=f"grouped_{name}", E=E, rows=R, H=H, F=F, ms=t, tflops=fl / t / 1e9,
                             frac_of_peak=fl / t / 1e9 / pk["tflops"], peak_src=pk["src"]))
            print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_elementwise():
    pk = peaks()
    rows = []
    T, H = 32768, 4096
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.randn(H, device="cuda").bfloat16()
    t, _ = time_fn(lambda: K.rmsnorm_fwd(x, w, 1e-6))
    rows.append(dict(op="rmsnorm_fwd", T=T, H=H, ms=t, gbs=2 * x.numel() * 2 / t / 1e6, frac=2 * x.numel() * 2 / t / 1e6 / pk["gbs"]))
    print(json.dumps(rows[-1]), flush=True)
    R, V = 4096, 151936
    lg = torch.randn(R, V, device="cuda").bfloat16()
    lab = torch.randint(0, V, (R,), device="cuda")
    t, _ = time_fn(lambda: K.cross_entropy(lg, lab, grad_out=lg))
    rows.append(dict(op="cross_entropy_fwd_bwd", R=R, V=V, ms=t, gbs=2 * lg.numel() * 2 / t / 1e6, frac=2 * lg.numel() * 2 / t / 1e6 / pk["gbs"]))
    print(json.dumps(rows[-1]), flush=True)
    xx = torch.randn(32768, 1536, device="cuda").bfloat16()
    t, _ = time_fn(lambda: K.swiglu_fwd(xx))
    rows.append(dict(op="swiglu_fwd", ms=t, gbs=xx.numel() * 3 / t / 1e6, frac=xx.numel() * 3 / t / 1e6 / pk["gbs"]))
    print(json.dumps(rows[-1]), flush=True)
    return rows


def profile_case(name: str) -> None:
    """One small, self-ending case per kernel for a profiler capture: inputs larger than L2 (126 MB) but well under
    a GB on the device, one warm-up launch and two more.  `python -m torchturbo_b200.benchmarks.kernel_bench
    profile:<gemm|grouped|grouped_dw|attn_fwd|attn_bwd|attn_mla|delta_state|adamw|rmsnorm>`."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape):
        return (torch.randn(*shape, device=dev, generator=g) * 0.1).bfloat16()

    if name == "gemm":
        a, b = rnd(8192, 4096), rnd(8192, 4096)                      # 64 MB + 64 MB in, 128 MB out
        fn = lambda: K.gemm(a, b)                                       # noqa: E731
    elif name == "grouped":
        E, H, F_, rows = 16, 2048, 768, 32768
        idx = torch.randint(0, E, (rows, 1), device=dev, dtype=torch.int32)
        pm = K.perm_index(idx, E)
        x = rnd(pm["capacity_rows"], H)
        w1 = rnd(E, H, 2 * F_)                                         # engine storage: [E, H, gate|up]
        fn = lambda: K.gemm(x, w1, b_mn=True, tile_group=pm["tile_group"], swiglu=True)   # noqa: E731
    elif name == "grouped_dw":
        # expert weight gradient at 1-GPU shapes: 128 experts x ~256 routed rows, dW[e] = x_e^T @ dy_e (bf16 out)
        E, H, F2, T, k = 128, 2048, 1536, 4096, 8
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32)
        pm = K.perm_index(idx, E)
        x, dy = rnd(pm["capacity_rows"], H), rnd(pm["capacity_rows"], F2)
        fn = lambda: K.gemm(x, dy, a_mn=True, b_mn=True, group_rows=pm["seg_start"])     # noqa: E731
    elif name in ("attn_fwd", "attn_bwd"):
        from ..ops.providers.b200_attention import FlashAttnFn

        T, Hq, Hk, D = 8192, 32, 8, 128
        q, k, v = rnd(T, Hq, D).requires_grad_(True), rnd(T, Hk, D).requires_grad_(True), rnd(T, Hk, D).requires_grad_(True)
        cu = torch.tensor([0, 3000, T], dtype=torch.int32)
        do = rnd(T, Hq, D)

        def fn():
            o = FlashAttnFn.apply(q, k, v, cu, 5192, True, D ** -0.5, False)
            if name == "attn_bwd":
                o.backward(do)
    elif name == "attn_mla":
        # multi-head latent attention widths: forward, kv-major backward (dK / dV) and the query-major dQ pass
        from ..ops.providers.b200_attention import FlashAttnFn

        T, H = 8192, 16
        q, k, v = rnd(T, H, 192).requires_grad_(True), rnd(T, H, 192).requires_grad_(True), rnd(T, H, 128).requires_grad_(True)
        cu = torch.tensor([0, 3000, T], dtype=torch.int32)
        do = rnd(T, H, 128)

        def fn():
            FlashAttnFn.apply(q, k, v, cu, 5192, True, 192 ** -0.5, False).backward(do)
    elif name == "delta_state":
        # recurrence over 64 chunks (4096 tokens) of 32 heads: 134 MB of states written, 67 MB of U read and X written
        H, NC = 32, 64
        a, b = rnd(H, NC, 64, 128), rnd(H, NC, 64, 128)
        u = torch.randn(H, NC, 64, 128, device=dev, generator=g)
        dec = torch.rand(H, NC, device=dev, generator=g)
        seq = torch.tensor([[0, NC]], dtype=torch.int32, device=dev)
        fn = lambda: K.delta_state_scan(a, b, u, dec, None, None, seq, reverse=False, s1=-1.0, s2=1.0)   # noqa: E731
    elif name == "adamw":
        n = 64 << 20                                                   # 64 Mi params: 256 MB each of p32, m, v, grad
        p16 = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        grad = torch.full((n,), 1e-3, device=dev, dtype=torch.bfloat16)
        p32, m, v2 = (torch.zeros(n, device=dev) for _ in range(3))
        plan = K.MultiTensorPlan([p32], [m], [v2], [p16])
        plan.refresh_grads([grad])
        step = [0]

        def fn():
            step[0] += 1
            K.adamw_step(plan, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=step[0])
    elif name in ("ulysses", "ep_dispatch"):
        # the peer-memory kernels on a 1-rank group: the "peer" is this GPU, so the counters show the kernels' own
        # memory behaviour (the NVLink leg needs 2+ ranks and cannot run under a profiler)
        import os

        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        if not dist.is_initialized():
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        if name == "ulysses":
            from ..comm import ulysses_p2p

            Tl, nq, nkv = 16384, 40, 8
            qkv = rnd(Tl, (nq + 2 * nkv) * 128)
            w = rnd(128) + 1.0
            pos = torch.arange(Tl, device=dev).float()
            inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device=dev).float() / 128))
            cos, sin = (pos[:, None] * inv[None]).cos(), (pos[:, None] * inv[None]).sin()

            def fn():
                q, k, v, ws = ulysses_p2p.qkv_exchange(qkv, nq, nkv, w, w, cos, sin, 1e-6, dist.group.WORLD)
                ulysses_p2p.out_exchange(q, ws)
        else:
            from ..comm.ep_p2p import P2PTokenDispatcher
            from ..models.modules.moe import MoELayerConfig

            T, H, E, k = 8192, 2048, 128, 8
            cfg = MoELayerConfig(hidden_size=H, moe_ffn_hidden_size=768, num_moe_experts=E, moe_router_topk=k,
                                 params_dtype=torch.bfloat16)
            disp = P2PTokenDispatcher(cfg, dist.group.WORLD, E)
            x = rnd(T, H)
            idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(64)]).repeat(T // 64, 1)
            prob = torch.rand(T, k, device=dev)

            def fn():
                perm, tpe, state = disp.dispatch(x, idx, prob)
                disp.combine(perm.tokens, state)
    elif name == "rmsnorm":
        x, w = rnd(32768, 4096), rnd(4096)
        fn = lambda: K.rmsnorm_fwd(x, w, 1e-6)                          # noqa: E731
    else:
        raise SystemExit(f"unknown profile case {name!r}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "launches": 3}))


def bench_delta_rule():
    """Gated delta rule, forward + backward of one layer: the chunk-parallel formulation with the `delta_state` kernel
    against the torch loop over chunks; the kernel alone for the recurrence time."""
    from ..ops.providers.b200_linear_attention import chunk_delta_rule_batched
    from ..ops.providers.native_linear_attention import chunk_delta_rule

    rows = []
    for T, H, vec in [(4096, 32, False), (4096, 8, True)]:
        D = 128
        q, k, v = (torch.randn(1, T, H, D, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
        g = (-torch.rand(1, T, H, *([D] if vec else []), device="cuda") * 0.3).requires_grad_(True)
        beta = torch.rand(1, T, H, device="cuda").requires_grad_(True)
        cu = [0, T]

        def run(fn):
            o, _ = fn(q, k, v, g, beta, cu_seqlens=cu, use_qk_l2norm=True)
            o.float().sum().backward()

        t_new, _ = time_fn(lambda: run(chunk_delta_rule_batched), iters=5, warmup=2)
        row = dict(op="delta_rule_fwd_bwd", T=T, H=H, vector_gate=vec, ms=t_new)
        if not vec:
            t_old, _ = time_fn(lambda: run(lambda *a, **kw: chunk_delta_rule(*a, **kw)), iters=2, warmup=1)
            row["torch_chunk_loop_ms"] = t_old
        NC = T // 64
        a = torch.randn(H, NC, 64, D, device="cuda").bfloat16() * 0.05
        u = torch.randn(H, NC, 64, D, device="cuda")
        dec = torch.rand(H, NC, device="cuda")
        seq = torch.tensor([[0, NC]], dtype=torch.int32, device="cuda")
        t_k, _ = time_fn(lambda: K.delta_state_scan(a, a, u, dec, None, None, seq, reverse=False, s1=-1.0, s2=1.0))
        row["state_kernel_ms"] = t_k
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


def main(argv):
    for a in argv:
        if a.startswith("profile:"):
            profile_case(a.split(":", 1)[1])
            return {}
    which = set(argv) or {"gemm", "grouped", "elementwise"}
    out = {}
    if "gemm" in which:
        out["gemm"] = bench_gemm()
    if "grouped" in which:
        out["grouped"] = bench_grouped()
    if "elementwise" in which:
        out["elementwise"] = bench_elementwise()
    if "attention" in which:
        from .attention_bench import bench_attention

        out["attention"] = bench_attention()
    if "delta" in which:
        out["delta"] = bench_delta_rule()
    return out


if __name__ == "__main__":
    main(sys.argv[1:])
