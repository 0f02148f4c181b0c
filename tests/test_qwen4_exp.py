"""Qwen4-Exp specifics: n-gram hashing rules, segment-aware halo convolution under sequence parallelism, QSA selection."""
import torch

from dist_utils import run_distributed
from torchturbo_b200.models.qwen4_exp.ple import NGramHasher, _conv_window, segment_causal_conv


def test_ngram_hash_isolation_and_eos_reset():
    h, total = NGramHasher.build(vocab=100, ngram_size=3, heads_per_ngram=2, base=50, ple_layer_index=0, seed=1, eos=0)
    assert h.head_sizes.tolist() == [53, 59, 61, 67] and total == 240 and h.head_offsets.tolist() == [0, 53, 112, 173]
    tok = torch.tensor([5, 6, 7, 0, 8, 9, 5, 6, 7])
    seg = torch.tensor([1, 1, 1, 1, 1, 1, 2, 2, 2])
    rows = h.row_ids(tok, seg)
    assert rows.shape == (9, 4) and (rows >= 0).all() and (rows < total).all()
    # the trigram (5,6,7) at position 2 and at position 8: same tokens, both with full in-sample history
    assert torch.equal(rows[2], rows[8])
    # position 6 starts sample 2: its history is EOS, exactly like a token right after an EOS (position 4 after the EOS at 3)
    solo = h.row_ids(torch.tensor([5]), torch.tensor([1]))
    assert torch.equal(rows[6], solo[0]) and torch.equal(rows[0], solo[0])
    after_eos = h.row_ids(torch.tensor([8]), torch.tensor([1]))
    assert torch.equal(rows[4], after_eos[0])
    # bigram heads of position 1 depend on tokens (6, 5) only
    again = h.row_ids(torch.tensor([5, 6]), torch.tensor([3, 3]))
    assert torch.equal(rows[1, :2], again[1, :2])


def _conv_ref(x, seg, w, dil):
    L, K = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(L):
        for k in range(K):
            src = t - (K - 1 - k) * dil
            if src >= 0 and seg[src] == seg[t]:
                y[t] += x[src] * w[:, k]
    return y


def test_conv_window_matches_loop():
    torch.manual_seed(0)
    x, w = torch.randn(20, 3), torch.randn(3, 3)
    seg = torch.tensor([1] * 7 + [2] * 9 + [0] * 4)
    assert torch.allclose(_conv_window(x, seg, w, 2), _conv_ref(x, seg, w, 2), atol=1e-6)


def _halo_worker(rank, world, out_dir):
    import torch.distributed as dist

    torch.manual_seed(0)
    T, C, K, dil = 24, 4, 3, 3                                  # history (K-1)*dil = 6 tokens, local length 12
    x_full, w = torch.randn(T, C), torch.randn(C, K)
    seg = torch.tensor([1] * 10 + [2] * 11 + [0] * 3)
    gy_full = torch.randn(T, C)
    xr, wr = x_full.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y_ref = segment_causal_conv(xr, wr, seg, dil)
    y_ref.backward(gy_full)
    Tl = T // world
    xl = x_full[rank * Tl:(rank + 1) * Tl].clone().requires_grad_(True)
    wl = w.clone().requires_grad_(True)
    y = segment_causal_conv(xl, wl, seg, dil, dist.group.WORLD, world, rank)
    y.backward(gy_full[rank * Tl:(rank + 1) * Tl])
    assert torch.allclose(y, y_ref[rank * Tl:(rank + 1) * Tl], atol=1e-5)
    assert torch.allclose(xl.grad, xr.grad[rank * Tl:(rank + 1) * Tl], atol=1e-5), (xl.grad - xr.grad[rank * Tl:(rank + 1) * Tl]).abs().max()
    gw = wl.grad.clone()
    dist.all_reduce(gw)
    assert torch.allclose(gw, wr.grad, atol=1e-4)


def test_halo_conv_sequence_parallel(tmp_path):
    run_distributed(_halo_worker, 2, str(tmp_path))


def test_qsa_selection_budget_and_tail():
    from types import SimpleNamespace

    from torchturbo_b200.models.modules.mixers import MixerContext
    from torchturbo_b200.models.qwen4_exp.modeling import QSAIndexer

    cfg = SimpleNamespace(indexer_n_heads=2, indexer_head_dim=8, indexer_budget=4, indexer_compress_ratio=2, hidden_size=16,
                          rms_norm_eps=1e-6)
    torch.manual_seed(0)
    ix = QSAIndexer(cfg)
    torch.nn.init.normal_(ix.index_qk_proj.weight, std=0.5)
    T = 14
    x = torch.randn(T, 16)
    cu = torch.tensor([0, 9, 14], dtype=torch.int32)
    pos = torch.cat([torch.arange(9), torch.arange(5)]).float()
    inv = 1.0 / (10000 ** (torch.arange(0, 8, 2).float() / 8))
    ang = pos[:, None] * inv[None]
    ctx = MixerContext(ang.cos(), ang.sin(), cu, 9)
    sel = ix(x, ctx)
    assert sel.shape == (T, 4 + 1)
    for t in range(T):
        a = 0 if t < 9 else 9
        ids = sel[t][sel[t] >= 0].tolist()
        assert all(a <= i <= t for i in ids) and len(set(ids)) == len(ids)    # causal, in-sample, no duplicates
        complete = (t - a + 1) // 2
        if complete <= 2 or (t - a + 1) % 2:
            assert t in ids                                                   # in the tail, or every block fits the budget
        assert len(ids) == min(complete, 2) * 2 + (t - a + 1 - complete * 2)  # whole blocks (budget 2) + causal tail
