"""Packed-row construction (`data/packing.py`): the batch contract, padding, the collator and the seeded synthetic dataset."""
import torch

from torchturbo_b200.data.packing import IGNORE_INDEX, PackedCollator, SyntheticPackedDataset, pack_documents


def test_packed_row_obeys_the_batch_contract():
    docs = [{"input_ids": [5, 6, 7], "labels": [IGNORE_INDEX, IGNORE_INDEX, 7]}, {"input_ids": []}, {"input_ids": [8, 9]}]
    b = pack_documents(docs)
    assert b["input_ids"].tolist() == [[5, 6, 7, 8, 9]]
    assert b["labels"].tolist() == [[IGNORE_INDEX, IGNORE_INDEX, 7, IGNORE_INDEX, 9]]     # first label of every document masked
    assert b["position_ids"].tolist() == [[0, 1, 2, 0, 1]]
    assert b["cu_seq_lens_q"].tolist() == [0, 3, 5] and b["cu_seq_lens_q"].dtype == torch.int32
    assert b["cu_seq_lens_k"] is not b["cu_seq_lens_q"] and torch.equal(b["cu_seq_lens_k"], b["cu_seq_lens_q"])
    assert b["max_length_q"] == b["max_length_k"] == 3 and "attention_mask" not in b


def test_padding_goes_behind_the_last_boundary():
    b = pack_documents([{"input_ids": [1, 2, 3]}], pad_to=8, pad_token_id=99)
    assert b["input_ids"].tolist() == [[1, 2, 3, 99, 99, 99, 99, 99]]
    assert b["labels"][0, 3:].eq(IGNORE_INDEX).all() and b["cu_seq_lens_q"].tolist() == [0, 3]
    assert pack_documents([{"input_ids": [1, 2, 3]}], pad_to=2)["input_ids"].shape == (1, 3)   # never truncates
    empty = pack_documents([], pad_to=4)
    assert empty["cu_seq_lens_q"].tolist() == [0] and empty["max_length_q"] == 0


def test_collator_flattens_samples_that_carry_several_documents():
    col = PackedCollator(pad_to=10)
    b = col([{"documents": [{"input_ids": [1, 2]}, {"input_ids": [3]}]}, {"input_ids": [4, 5, 6]}])
    assert b["cu_seq_lens_q"].tolist() == [0, 2, 3, 6] and b["input_ids"].shape == (1, 10)


def test_synthetic_dataset_is_seeded_and_fills_the_row():
    ds = SyntheticPackedDataset(4, 1000, 50, min_doc=100, max_doc=300, seed=3)
    assert len(ds) == 4
    lens = ds.doc_lengths(2)
    assert sum(lens) == 1000 and all(1 <= n <= 300 for n in lens) and all(n >= 100 for n in lens[:-1])
    a, b = ds[2], SyntheticPackedDataset(4, 1000, 50, min_doc=100, max_doc=300, seed=3)[2]
    assert a == b and ds[1] != ds[2]
    row = PackedCollator()([ds[2]])
    assert row["input_ids"].shape == (1, 1000) and int(row["input_ids"].max()) < 50
    fixed = SyntheticPackedDataset(2, 512, 50, num_docs=5, seed=1)
    assert len(fixed.doc_lengths(0)) == 5 and sum(fixed.doc_lengths(0)) == 512
