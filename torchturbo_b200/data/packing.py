"""Packed-batch construction: several documents flattened into one row `[1, T]` with `cu_seq_lens`.

The contract every training batch obeys (engine/utils.py:142-198 and the collators of the reference's adapters):
`input_ids [1,T]`, `labels [1,T]` (unshifted; the first label of every document is -100), `position_ids [1,T]`
restarting at 0 per document, `cu_seq_lens_q == cu_seq_lens_k` (CPU int32), `max_length_q == max_length_k`
(Python int), and no `attention_mask`."""
from __future__ import annotations

from typing import Any, Iterable, Sequence

import torch
from torch.utils.data import Dataset

IGNORE_INDEX = -100


def pack_documents(docs: Sequence[dict[str, Sequence[int]]], *, pad_to: int | None = None, pad_token_id: int = 0,
                   pin: bool = False) -> dict[str, Any]:
    """docs: [{"input_ids": [...], "labels": [...] (optional)}] -> one packed row."""
    ids, labels, pos, cu = [], [], [], [0]
    for d in docs:
        x = list(d["input_ids"])
        y = list(d.get("labels", x))
        if len(x) == 0:
            continue
        y = [IGNORE_INDEX] + y[1:]
        ids += x
        labels += y
        pos += list(range(len(x)))
        cu.append(cu[-1] + len(x))
    T = len(ids)
    if pad_to is not None and T < pad_to:
        n = pad_to - T
        ids += [pad_token_id] * n
        labels += [IGNORE_INDEX] * n
        pos += list(range(n))
    mx = max((b - a for a, b in zip(cu[:-1], cu[1:])), default=0)
    cu_t = torch.tensor(cu, dtype=torch.int32)
    batch = {
        "input_ids": torch.tensor(ids, dtype=torch.long).unsqueeze(0),
        "labels": torch.tensor(labels, dtype=torch.long).unsqueeze(0),
        "position_ids": torch.tensor(pos, dtype=torch.long).unsqueeze(0),
        "cu_seq_lens_q": cu_t, "cu_seq_lens_k": cu_t.clone(),
        "max_length_q": mx, "max_length_k": mx,
    }
    if pin and torch.cuda.is_available():
        for k in ("input_ids", "labels", "position_ids"):
            batch[k] = batch[k].pin_memory()
    return batch


class PackedCollator:
    """Collate a list of tokenised samples into one packed row (micro-batch size in rows is always 1)."""

    def __init__(self, pad_to: int | None = None, pad_token_id: int = 0, pin: bool = False):
        self.pad_to, self.pad_token_id, self.pin = pad_to, pad_token_id, pin

    def __call__(self, samples: Iterable[dict]) -> dict[str, Any]:
        docs = []
        for s in samples:
            if "documents" in s:
                docs += list(s["documents"])
            else:
                docs.append(s)
        return pack_documents(docs, pad_to=self.pad_to, pad_token_id=self.pad_token_id, pin=self.pin)


class SyntheticPackedDataset(Dataset):
    """Seeded synthetic packs: every item is `seq_len` tokens made of documents with random lengths in
    `[min_doc, max_doc]` (the last one truncated to fit) and uniform random token ids."""

    def __init__(self, num_samples: int, seq_len: int, vocab_size: int, *, min_doc: int = 256, max_doc: int | None = None,
                 num_docs: int | None = None, seed: int = 0):
        self.n, self.seq_len, self.vocab = num_samples, seq_len, vocab_size
        self.min_doc, self.max_doc, self.num_docs, self.seed = min_doc, max_doc or seq_len, num_docs, seed

    def __len__(self) -> int:
        return self.n

    def doc_lengths(self, i: int) -> list[int]:
        g = torch.Generator().manual_seed(self.seed * 1000003 + i)
        if self.num_docs:
            cuts = sorted(torch.randperm(self.seq_len - 1, generator=g)[: self.num_docs - 1].add(1).tolist())
            edges = [0] + cuts + [self.seq_len]
            return [b - a for a, b in zip(edges[:-1], edges[1:])]
        lens, left = [], self.seq_len
        while left > 0:
            L = int(torch.randint(self.min_doc, self.max_doc + 1, (1,), generator=g))
            L = min(L, left)
            lens.append(L)
            left -= L
        return lens

    def __getitem__(self, i: int) -> dict:
        g = torch.Generator().manual_seed(self.seed * 7919 + i)
        docs = []
        for L in self.doc_lengths(i):
            ids = torch.randint(0, self.vocab, (L,), generator=g).tolist()
            docs.append({"input_ids": ids, "labels": ids})
        return {"documents": docs}
