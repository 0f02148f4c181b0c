"""Chunk-parallel formulation of the (gated) delta rule with the recurrence over chunks factored out
(`ops/providers/b200_linear_attention.py`): against the token-by-token oracle on CPU, where the recurrence runs as a
torch loop, and on a GPU, where it runs on the `delta_state` kernel (forward and the reverse pass)."""
import pytest
import torch

from torchturbo_b200.ops.providers.b200_linear_attention import _scan_torch, chunk_delta_rule_batched
from torchturbo_b200.ops.providers.native_linear_attention import delta_rule_recurrent, l2norm


def _inputs(T, H, Kd, V, vec, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, T, H, Kd, generator=g)
    k = torch.randn(1, T, H, Kd, generator=g)
    v = torch.randn(1, T, H, V, generator=g)
    gate = -torch.rand(1, T, H, *([Kd] if vec else []), generator=g) * 0.3
    beta = torch.rand(1, T, H, generator=g)
    return [t.to(device) for t in (q, k, v, gate, beta)]


@pytest.mark.parametrize("vec", [False, True])
def test_batched_chunks_match_the_recurrent_oracle_on_ragged_sequences(vec):
    T, H, Kd, V = 300, 2, 16, 24
    q, k, v, g, beta = _inputs(T, H, Kd, V, vec)
    cu = [0, 70, 70, 199, 300]                       # one empty sequence, none a multiple of the chunk
    init = torch.randn(4, H, Kd, V) * 0.1
    qn, kn = l2norm(q), l2norm(k)
    want, want_S = delta_rule_recurrent(qn, kn, v, g, beta, initial_state=init, cu_seqlens=cu)
    got, got_S = chunk_delta_rule_batched(q, k, v, g, beta, initial_state=init, output_final_state=True, cu_seqlens=cu,
                                          use_qk_l2norm=True)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
    assert torch.allclose(got_S, want_S, atol=2e-4, rtol=1e-3)
    assert torch.equal(got_S[1], init[1])            # the empty sequence hands its initial state through


def test_reverse_scan_is_the_gradient_of_the_forward_scan():
    """The contract the kernel's backward relies on: running the recurrence in reverse with (k_out, w) swapped gives the
    gradients that autograd finds for the forward loop."""
    torch.manual_seed(1)
    H, NC, C, Kd, V = 2, 5, 8, 6, 7
    seq = [(0, 2), (2, 0), (2, 3)]
    u, w, ko = (torch.randn(H, NC, C, d, dtype=torch.float64, requires_grad=True) for d in (V, Kd, Kd))
    decay = torch.rand(H, NC, dtype=torch.float64).requires_grad_(True)
    init = torch.randn(H, 3, Kd, V, dtype=torch.float64, requires_grad=True)
    x, states = _scan_torch(u, w, ko, decay, init, seq)
    gx, gs = torch.randn_like(x), torch.randn_like(states)
    (x * gx).sum().add((states * gs).sum()).backward()
    with torch.no_grad():
        dx, dS = _scan_torch(gx, ko, w, decay, None, seq, reverse=True, add=gs, s1=1.0, s2=-1.0)
        start = torch.tensor([c + s for s, (c0, n) in enumerate(seq) for c in range(c0, c0 + n)])
        S_c, dS_n = states.index_select(1, start), dS.index_select(1, start + 1)
        assert torch.allclose(dx, u.grad)
        assert torch.allclose(-(dx @ S_c.transpose(-1, -2)), w.grad)
        assert torch.allclose(x @ dS_n.transpose(-1, -2), ko.grad)
        assert torch.allclose((dS_n * S_c).sum((-1, -2)), decay.grad)
        first = torch.tensor([c0 + s for s, (c0, n) in enumerate(seq)])
        assert torch.allclose(dS.index_select(1, first), init.grad)


@pytest.mark.gpu
@pytest.mark.parametrize("vec", [False, True])
def test_delta_state_kernel_matches_the_oracle_forward_and_backward(vec):
    from torchturbo_b200 import kernels as K

    T, H, D = 700, 3, 128
    q, k, v, g, beta = _inputs(T, H, D, D, vec, device="cuda", seed=2)
    cu = [0, 130, 131, 520, 700]
    init = (torch.randn(4, H, D, D, device="cuda") * 0.05).requires_grad_(True)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    before = K.launch_count()
    out, fin = chunk_delta_rule_batched(*leaves, initial_state=init, output_final_state=True, cu_seqlens=cu, use_qk_l2norm=True)
    assert K.launch_count() > before
    go, gf = torch.randn_like(out), torch.randn_like(fin) * 0.1
    (out * go).sum().add((fin * gf).sum()).backward()
    torch.cuda.synchronize()
    assert K.status() == (0, 0)
    # oracle: the same formulation with the recurrence as an fp32 torch loop on the CPU
    ref_leaves = [t.detach().cpu().clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    init_c = init.detach().cpu().clone().requires_grad_(True)
    ro, rf = chunk_delta_rule_batched(*ref_leaves, initial_state=init_c, output_final_state=True, cu_seqlens=cu, use_qk_l2norm=True)
    (ro * go.cpu()).sum().add((rf * gf.cpu()).sum()).backward()
    want, _ = delta_rule_recurrent(l2norm(q.cpu()), l2norm(k.cpu()), v.cpu(), g.cpu(), beta.cpu(), initial_state=init_c.detach(),
                                   cu_seqlens=cu)
    assert torch.allclose(ro, want, atol=5e-4, rtol=1e-3)

    def close(a, b, what):
        err = (a.cpu().float() - b.float()).abs().max().item()
        ref = b.float().abs().max().item()
        assert err <= 2e-2 * max(ref, 1.0), f"{what}: {err} vs {ref}"      # bf16 operands inside the recurrence

    close(out, ro, "output")
    close(fin, rf, "final state")
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta"), leaves, ref_leaves):
        close(a.grad, b.grad, name)
    close(init.grad, init_c.grad, "dinit")


def test_chunk_aligned_rows_take_the_view_path_and_a_padded_tail_is_one_more_sequence():
    T, H, Kd, V = 256, 2, 16, 16
    q, k, v, g, beta = _inputs(T, H, Kd, V, False, seed=4)
    qn, kn = l2norm(q), l2norm(k)
    for cu in ([0, 128, 256], [0, 100, 200]):             # whole chunks (a view) / ragged with rows behind the last boundary
        want, _ = delta_rule_recurrent(qn, kn, v, g, beta, cu_seqlens=cu)
        got, _ = chunk_delta_rule_batched(q, k, v, g, beta, cu_seqlens=cu, use_qk_l2norm=True)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), cu


@pytest.mark.gpu
def test_gated_delta_net_mixer_on_cuda_runs_the_state_kernel_and_matches_the_cpu_module():
    """The Qwen3.5 mixer through the operator dispatcher: on CUDA `ops.gated_delta_rule` resolves to the provider with
    the `delta_state` kernel; output and parameter gradients against the same module on the CPU in fp32."""
    from types import SimpleNamespace

    from torchturbo_b200 import kernels as K
    from torchturbo_b200.models.modules.mixers import GatedDeltaNet, MixerContext
    from torchturbo_b200.ops import OpDispatcher, OpPolicy

    assert type(OpDispatcher(OpPolicy.AUTO).resolve("gated_delta_rule")).__name__ == "B200GatedDeltaRule"
    cfg = SimpleNamespace(hidden_size=256, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128,
                          linear_value_head_dim=128, linear_conv_kernel_dim=4, rms_norm_eps=1e-6, hidden_act="silu")
    torch.manual_seed(0)
    ref = GatedDeltaNet(cfg, 0).float()
    dev = GatedDeltaNet(cfg, 0).float()
    dev.load_state_dict(ref.state_dict())
    dev = dev.cuda()
    T = 200
    x = torch.randn(T, 256) * 0.5
    cu = torch.tensor([0, 70, 200], dtype=torch.int32)
    ctx_c = ctx_g = MixerContext(cos=None, sin=None, cu_seqlens=cu, max_seqlen=130)
    want = ref(x, ctx_c)
    want.square().sum().backward()
    before = K.launch_count()
    got = dev(x.cuda(), ctx_g)
    got.square().sum().backward()
    torch.cuda.synchronize()
    assert K.launch_count() > before and K.status() == (0, 0)
    assert (got.cpu() - want).abs().max() <= 2e-2 * max(1.0, want.abs().max())
    for (n, a), b in zip(dev.named_parameters(), ref.parameters()):
        assert (a.grad.cpu() - b.grad).abs().max() <= 3e-2 * max(1.0, b.grad.abs().max()), n
