"""Seeded synthetic vision-language rows for benchmarks and tests.

One item = one packed row of one sample: `text_len` random text tokens with, for every image, a run of image
placeholder tokens (one per merged patch, preceded by the vision-start token) inserted at a seeded position, plus the
packed patches of all images.  Image count is uniform in `[min_images, max_images]`; height and width are uniform in
`[min_side, max_side]` pixels rounded to a multiple of `patch * merge` (28 for the Qwen-VL tower), pixels are
normal(0, 1).  A rank may get zero images: the vision balancer then feeds it pooled images of other ranks (or the
model's dummy image), which is the case the rebalancing exists for."""
from __future__ import annotations

import torch
from torch.utils.data import Dataset

from .packing import IGNORE_INDEX


class SyntheticVLMDataset(Dataset):
    def __init__(self, num_samples: int, text_len: int, vocab_size: int, *, image_token_id: int, vision_start_token_id: int,
                 min_images: int = 0, max_images: int = 8, min_side: int = 224, max_side: int = 1344, patch: int = 14,
                 merge: int = 2, temporal_patch: int = 2, channels: int = 3, max_row_tokens: int | None = None, seed: int = 0):
        self.n, self.text_len, self.vocab = num_samples, text_len, vocab_size
        self.img_tok, self.start_tok = image_token_id, vision_start_token_id
        self.min_images, self.max_images, self.min_side, self.max_side = min_images, max_images, min_side, max_side
        self.patch, self.merge, self.tp, self.ch = patch, merge, temporal_patch, channels
        self.max_row_tokens, self.seed = max_row_tokens, seed

    def __len__(self) -> int:
        return self.n

    def grids(self, i: int) -> list[tuple[int, int, int]]:
        """(t, h, w) patch grids of the images of item i."""
        g = torch.Generator().manual_seed(self.seed * 104729 + i)
        k = int(torch.randint(self.min_images, self.max_images + 1, (1,), generator=g))
        unit = self.patch * self.merge
        out, budget = [], (self.max_row_tokens - self.text_len) if self.max_row_tokens else None
        for _ in range(k):
            h, w = (int(torch.randint(self.min_side, self.max_side + 1, (1,), generator=g)) // unit * unit for _ in range(2))
            gh, gw = max(h, unit) // self.patch, max(w, unit) // self.patch
            need = gh * gw // (self.merge ** 2) + 1
            if budget is not None:
                if need > budget:
                    continue
                budget -= need
            out.append((1, gh, gw))
        return out

    def __getitem__(self, i: int) -> dict:
        g = torch.Generator().manual_seed(self.seed * 7919 + i)
        grids = self.grids(i)
        text = torch.randint(0, min(self.vocab, self.img_tok), (self.text_len,), generator=g)
        cuts = sorted(torch.randint(1, self.text_len, (len(grids),), generator=g).tolist())
        pieces, labels, prev = [], [], 0
        for (t, h, w), c in zip(grids, cuts):
            n_tok = t * h * w // (self.merge ** 2)
            pieces += [text[prev:c], torch.tensor([self.start_tok]), torch.full((n_tok,), self.img_tok)]
            labels += [text[prev:c], torch.full((n_tok + 1,), IGNORE_INDEX)]
            prev = c
        pieces.append(text[prev:])
        labels.append(text[prev:])
        ids, lab = torch.cat(pieces), torch.cat(labels).clone()
        lab[0] = IGNORE_INDEX
        T = ids.numel()
        n_patches = sum(t * h * w for t, h, w in grids)
        feat = self.ch * self.tp * self.patch * self.patch
        cu = torch.tensor([0, T], dtype=torch.int32)
        return {
            "input_ids": ids[None], "labels": lab[None], "position_ids": torch.arange(T)[None],
            "cu_seq_lens_q": cu, "cu_seq_lens_k": cu.clone(), "max_length_q": T, "max_length_k": T,
            "pixel_values": torch.randn(n_patches, feat, generator=g).to(torch.bfloat16),
            "image_grid_thw": torch.tensor(grids, dtype=torch.long).reshape(-1, 3),
        }
