"""Loss streams (label shifting across document boundaries, normalisers under sequence parallelism, chunked projection +
cross entropy) and the host-side tile tables of the attention kernels."""
import pytest
import torch
import torch.nn.functional as F

from torchturbo_b200 import kernels as K
from torchturbo_b200.models.modules.loss.lm_loss import IGNORE_INDEX, chunk_loss, logits_loss, prepare_loss_labels, shift_labels_packed


def test_shift_never_crosses_a_document_boundary_and_padding_is_ignored():
    labels = torch.arange(100, 112)[None]                       # 12 rows: documents [0,5), [5,9), padding 9..11
    cu = torch.tensor([0, 5, 9])
    s1 = shift_labels_packed(labels, cu, 1)[0].tolist()
    assert s1 == [101, 102, 103, 104, IGNORE_INDEX, 106, 107, 108, IGNORE_INDEX, IGNORE_INDEX, IGNORE_INDEX, IGNORE_INDEX]
    s2 = shift_labels_packed(labels, cu, 2)[0].tolist()
    assert s2 == [102, 103, 104, IGNORE_INDEX, IGNORE_INDEX, 107, 108, IGNORE_INDEX, IGNORE_INDEX, IGNORE_INDEX, IGNORE_INDEX,
                  IGNORE_INDEX]
    assert shift_labels_packed(labels, cu, 50)[0].eq(IGNORE_INDEX).all()


def test_masked_prompt_labels_stay_masked_after_the_shift():
    labels = torch.tensor([[IGNORE_INDEX, IGNORE_INDEX, 7, 8, IGNORE_INDEX, 9]])
    out = shift_labels_packed(labels, torch.tensor([0, 4, 6]), 1)[0].tolist()
    assert out == [IGNORE_INDEX, 7, 8, IGNORE_INDEX, 9, IGNORE_INDEX]


@pytest.mark.parametrize("sp", [1, 2, 4])
def test_sequence_parallel_slices_add_up_to_the_full_row_loss(sp):
    torch.manual_seed(0)
    T, V = 16, 11
    labels = torch.randint(0, V, (1, T))
    labels[0, :3] = IGNORE_INDEX
    cu = torch.tensor([0, 7, 16])
    logits = torch.randn(1, T, V)
    full_streams = prepare_loss_labels(labels, cu)
    want, _ = logits_loss(logits, full_streams)
    shifted = shift_labels_packed(labels, cu, 1)
    direct = F.cross_entropy(logits[0], shifted[0], ignore_index=IGNORE_INDEX, reduction="sum") / (shifted != IGNORE_INDEX).sum()
    assert torch.allclose(want, direct, atol=1e-6)
    local = T // sp
    # every rank normalises by (valid labels of the row) * sp: the ranks' losses add up to 1 / sp of the row loss (the
    # gradient all-reduce over the sp group, which averages over data-parallel ranks only, restores the factor)
    parts = []
    for r in range(sp):
        st = prepare_loss_labels(labels, cu, sp_size=sp, sp_rank=r)
        assert st[0].labels.shape[-1] == local
        parts.append(logits_loss(logits[:, r * local:(r + 1) * local], st)[0])
    assert torch.allclose(torch.stack(parts).sum() * sp, want, atol=1e-6)


def test_global_token_count_normaliser_is_floored_to_the_sequence_parallel_size():
    labels = torch.randint(0, 5, (1, 8))
    st = prepare_loss_labels(labels, torch.tensor([0, 8]), num_items_in_batch=103, sp_size=4, sp_rank=1, world_size=8)
    assert st[0].normalizer == (103 // 4) * 4 / 8
    st = prepare_loss_labels(labels, torch.tensor([0, 8]), num_items_in_batch=torch.tensor(103), sp_size=4, sp_rank=0, world_size=8)
    assert float(st[0].normalizer) == (103 // 4) * 4 / 8


def test_prediction_depth_streams_shift_further_and_weigh_into_the_total():
    torch.manual_seed(1)
    T, V, H = 12, 9, 6
    labels = torch.randint(0, V, (1, T))
    cu = torch.tensor([0, 5, 12])
    streams = prepare_loss_labels(labels, cu, num_streams=3, stream_scales=[1.0, 0.3, 0.0])
    assert [s.name for s in streams] == ["main", "mtp1", "mtp2"]
    assert torch.equal(streams[1].labels, shift_labels_packed(labels, cu, 2))
    hidden = [torch.randn(1, T, H) for _ in range(3)]
    w = torch.randn(V, H)
    total, comps = chunk_loss(hidden, w, streams, chunk_size=5)
    want = []
    for h, st in zip(hidden, streams):
        ce = F.cross_entropy(h[0] @ w.t(), st.labels[0], ignore_index=IGNORE_INDEX, reduction="sum")
        want.append(ce / (st.labels != IGNORE_INDEX).sum().clamp(min=1))
    assert torch.allclose(total, want[0] + 0.3 * want[1], atol=1e-5)
    assert set(comps) == {"main", "mtp1", "mtp2"} and torch.allclose(comps["mtp2"], want[2], atol=1e-5)


def test_chunked_projection_loss_has_the_gradients_of_the_full_one():
    torch.manual_seed(2)
    T, V, H = 37, 23, 8
    h1 = torch.randn(1, T, H, requires_grad=True)
    w1 = torch.randn(V, H, requires_grad=True)
    h2, w2 = h1.detach().clone().requires_grad_(True), w1.detach().clone().requires_grad_(True)
    labels = torch.randint(0, V, (1, T))
    labels[0, 5:9] = IGNORE_INDEX
    streams = prepare_loss_labels(labels, torch.tensor([0, 20, 37]))
    a, _ = chunk_loss(h1, w1, streams, chunk_size=8)
    b, _ = logits_loss(h2 @ w2.t(), streams)
    a.backward()
    b.backward()
    assert torch.allclose(a, b, atol=1e-6)
    assert torch.allclose(h1.grad, h2.grad, atol=1e-6) and torch.allclose(w1.grad, w2.grad, atol=1e-6)


@pytest.mark.parametrize("cu", [[0, 4096], [0, 130, 131, 600, 900], [0, 1], [0, 128, 256], [0, 0, 300]])
def test_attention_tile_tables_cover_every_token_once_and_start_with_the_longest_tiles(cu):
    for build in (K.build_q_tiles, K.build_kv_tiles):
        t = build(torch.tensor(cu, dtype=torch.int32))
        assert t.dtype == torch.int32 and t.shape[1] == 3
        seen = torch.zeros(cu[-1], dtype=torch.int32)
        for first, ds, de in t.tolist():
            assert ds <= first < de and (first - ds) % 128 == 0 and (ds, de) in set(zip(cu[:-1], cu[1:]))
            seen[first:min(first + 128, de)] += 1
        assert bool((seen == 1).all())
    q = K.build_q_tiles(torch.tensor(cu, dtype=torch.int32)).tolist()
    work_q = [first - ds for first, ds, de in q]                 # causal: kv blocks seen grow with the offset in the document
    assert work_q == sorted(work_q, reverse=True)
    kv = K.build_kv_tiles(torch.tensor(cu, dtype=torch.int32)).tolist()
    work_kv = [de - first for first, ds, de in kv]               # causal: query tiles that see a kv tile shrink with its offset
    assert work_kv == sorted(work_kv, reverse=True)
