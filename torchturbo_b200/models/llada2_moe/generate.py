"""Block-diffusion sampling for LLaDA2: the answer is produced one block of `block_size` tokens at a time; inside a
block all positions start as the mask token and, over `steps` denoising passes, the most confident predictions are
committed first (models/llada2_moe/generate.py of the reference follows the same schedule: confidence-ordered
unmasking with a per-step quota, earlier blocks frozen as context)."""
from __future__ import annotations

import torch

from .bd import SEG_CLEAN, block_diffusion_allow


@torch.no_grad()
def generate(model, prompt_ids: torch.Tensor, *, max_new_tokens: int = 128, block_size: int = 32, steps: int = 8,
             temperature: float = 0.0, mask_id: int | None = None, eos_id: int | None = None) -> torch.Tensor:
    """prompt_ids: [L] -> [L + n] token ids (n <= max_new_tokens, cut at the first `eos_id`)."""
    cfg = model.config
    mask_id = cfg.mask_token_id if mask_id is None else mask_id
    dev = prompt_ids.device
    seq = prompt_ids.reshape(-1).clone()
    n_blocks = (max_new_tokens + block_size - 1) // block_size
    for _ in range(n_blocks):
        start = seq.numel()
        # committed tokens are "clean" context; blocks are counted from the start of the row so the new block is one unit
        cur = torch.cat((seq, torch.full((block_size,), mask_id, dtype=seq.dtype, device=dev)))
        T = cur.numel()
        pos = torch.arange(T, device=dev)
        block = torch.where(pos < start, pos // block_size, torch.full_like(pos, (start + block_size - 1) // block_size + 1))
        allow = block_diffusion_allow(torch.zeros(T, dtype=torch.long, device=dev),
                                      torch.full((T,), SEG_CLEAN, dtype=torch.long, device=dev), block)
        open_ = torch.ones(block_size, dtype=torch.bool, device=dev)
        for s in range(steps):
            logits = model(input_ids=cur.unsqueeze(0), position_ids=pos.unsqueeze(0), block_allow=allow).logits[0, start:]
            if temperature > 0:
                probs = torch.softmax(logits.float() / temperature, -1)
                pick = torch.multinomial(probs, 1).squeeze(-1)
                conf = probs.gather(-1, pick[:, None]).squeeze(-1)
            else:
                probs = torch.softmax(logits.float(), -1)
                conf, pick = probs.max(-1)
            conf = conf.masked_fill(~open_, -1.0)
            quota = int(open_.sum()) if s == steps - 1 else max(1, (int(open_.sum()) + (steps - s) - 1) // (steps - s))
            take = conf.topk(min(quota, int(open_.sum()))).indices
            cur[start + take] = pick[take].to(cur.dtype)
            open_[take] = False
            if not bool(open_.any()):
                break
        seq = cur
        if eos_id is not None and bool((seq[start:] == eos_id).any()):
            cut = start + int((seq[start:] == eos_id).nonzero()[0]) + 1
            return seq[:cut]
    return seq[: prompt_ids.numel() + max_new_tokens]
