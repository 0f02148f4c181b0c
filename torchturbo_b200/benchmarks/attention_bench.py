"""Device-timed comparison of the tcgen05 varlen attention with flash-attn 2 (library baseline)."""
from __future__ import annotations

import json

import torch

from .. import kernels as K
from .kernel_bench import peaks, time_fn


def bench_attention():
    pk = peaks()
    rows = []
    for T, Hq, Hk, docs in [(4096, 32, 4, [4096]), (8192, 32, 8, [8192]), (8192, 32, 8, [1000, 3000, 4192]),
                            (65536, 5, 1, [65536])]:
        D = 128
        q = torch.randn(T, Hq, D, device="cuda").bfloat16()
        k = torch.randn(T, Hk, D, device="cuda").bfloat16()
        v = torch.randn(T, Hk, D, device="cuda").bfloat16()
        cu = torch.tensor([0] + list(torch.tensor(docs).cumsum(0)), dtype=torch.int32)
        tiles = K.build_q_tiles(cu).cuda()
        fl = sum(4.0 * L * L * Hq * D / 2 for L in docs)
        t, _ = time_fn(lambda: K.attn_fwd(q, k, v, tiles, scale=D ** -0.5, causal=True))
        row = dict(op="attn_fwd_causal", T=T, Hq=Hq, Hk=Hk, docs=docs, ms=t, tflops=fl / t / 1e9,
                   frac_of_peak=fl / t / 1e9 / pk["tflops"], peak_src=pk["src"])
        try:
            from flash_attn import flash_attn_varlen_func

            cud = cu.cuda()
            mx = max(docs)
            t2, _ = time_fn(lambda: flash_attn_varlen_func(q, k, v, cud, cud, mx, mx, causal=True))
            row["flash_attn2_ms"] = t2
            row["flash_attn2_tflops"] = fl / t2 / 1e9
        except Exception as e:  # noqa: BLE001
            row["flash_attn2_error"] = str(e)[:80]
        rows.append(row)
        print(json.dumps(row), flush=True)
        # backward: the whole call (row dot products, the tcgen05 kernel, fp32 -> bf16 casts of dQ / dK / dV)
        out, lse, _ = K.attn_fwd(q, k, v, tiles, scale=D ** -0.5, causal=True)
        dout = torch.randn_like(out)
        kv_tiles = K.build_kv_tiles(cu).cuda()
        tb, _ = time_fn(lambda: K.attn_bwd(dout, q, k, v, out, lse, kv_tiles, scale=D ** -0.5, causal=True))
        rowb = dict(op="attn_bwd_causal", T=T, Hq=Hq, Hk=Hk, docs=docs, ms=tb, tflops=2.5 * fl / tb / 1e9,
                    frac_of_peak=2.5 * fl / tb / 1e9 / pk["tflops"], peak_src=pk["src"])
        try:
            from flash_attn import flash_attn_varlen_func

            qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            o2 = flash_attn_varlen_func(qg, kg, vg, cud, cud, mx, mx, causal=True)
            t3, _ = time_fn(lambda: torch.autograd.grad(o2, (qg, kg, vg), dout, retain_graph=True))
            rowb["flash_attn2_ms"] = t3
        except Exception as e:  # noqa: BLE001
            rowb["flash_attn2_error"] = str(e)[:80]
        rows.append(rowb)
        print(json.dumps(rowb), flush=True)
        td, _ = time_fn(lambda: K.attn_bwd(dout, q, k, v, out, lse, kv_tiles, scale=D ** -0.5, causal=True, q_tiles_dev=tiles,
                                          deterministic=True))
        rowd = dict(op="attn_bwd_causal_deterministic", T=T, Hq=Hq, Hk=Hk, docs=docs, ms=td, tflops=2.5 * fl / td / 1e9,
                    frac_of_peak=2.5 * fl / td / 1e9 / pk["tflops"], peak_src=pk["src"])
        rows.append(rowd)
        print(json.dumps(rowd), flush=True)
    # multi-head latent attention: query / key heads 192 wide, value heads 128 wide, no grouped-query sharing
    for T, H, docs in [(4096, 16, [4096]), (8192, 16, [8192])]:
        q = torch.randn(T, H, 192, device="cuda").bfloat16()
        k = torch.randn(T, H, 192, device="cuda").bfloat16()
        v = torch.randn(T, H, 128, device="cuda").bfloat16()
        cu = torch.tensor([0] + list(torch.tensor(docs).cumsum(0)), dtype=torch.int32)
        tiles, kv_tiles = K.build_q_tiles(cu).cuda(), K.build_kv_tiles(cu).cuda()
        fl = sum(2.0 * L * L * H * (192 + 128) / 2 for L in docs)
        sc = 192 ** -0.5
        t, _ = time_fn(lambda: K.attn_fwd(q, k, v, tiles, scale=sc, causal=True))
        out, lse, _ = K.attn_fwd(q, k, v, tiles, scale=sc, causal=True)
        dout = torch.randn_like(out)
        tb, _ = time_fn(lambda: K.attn_bwd(dout, q, k, v, out, lse, kv_tiles, scale=sc, causal=True, q_tiles_dev=tiles))
        row = dict(op="mla_attn_fwd_bwd_causal", T=T, H=H, docs=docs, fwd_ms=t, bwd_ms=tb, fwd_tflops=fl / t / 1e9,
                   bwd_tflops=2.5 * fl / tb / 1e9, fwd_frac_of_peak=fl / t / 1e9 / pk["tflops"],
                   bwd_frac_of_peak=2.5 * fl / tb / 1e9 / pk["tflops"], peak_src=pk["src"])
        try:
            from flash_attn import flash_attn_varlen_func

            # the library wants equal head widths: values zero-padded to 192 columns, as the library provider does
            cud, mx = cu.cuda(), max(docs)
            qg, kg = (x.detach().clone().requires_grad_(True) for x in (q, k))
            vg = torch.nn.functional.pad(v, (0, 64)).requires_grad_(True)
            dpad = torch.nn.functional.pad(dout, (0, 64))
            t2, _ = time_fn(lambda: flash_attn_varlen_func(qg, kg, vg, cud, cud, mx, mx, softmax_scale=sc, causal=True))
            o2 = flash_attn_varlen_func(qg, kg, vg, cud, cud, mx, mx, softmax_scale=sc, causal=True)
            t3, _ = time_fn(lambda: torch.autograd.grad(o2, (qg, kg, vg), dpad, retain_graph=True))
            row["flash_attn2_fwd_ms"], row["flash_attn2_bwd_ms"] = t2, t3
        except Exception as e:  # noqa: BLE001
            row["flash_attn2_error"] = str(e)[:80]
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows
