"""Token choice from a row of logits: greedy arg-max or temperature / top-k / top-p sampling.
Shared by every decode loop of the package (HF `generate` semantics, llava_arch.py:802-821)."""
from __future__ import annotations

from typing import Optional

import torch


def pick_token(logits: torch.Tensor, sample: bool = False, temperature: float = 1.0, top_k: int = 0,
               top_p: float = 1.0, generator: Optional[torch.Generator] = None) -> int:
    """logits [V] (any float dtype) -> token id."""
    lg = logits.float()
    if not sample:
        return int(torch.argmax(lg))
    lg = lg / max(temperature, 1e-5)
    if top_k and top_k > 0:
        kth = torch.topk(lg, min(top_k, lg.numel())).values[-1]
        lg = lg.masked_fill(lg < kth, float("-inf"))
    probs = torch.softmax(lg, -1)
    if top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cut = torch.cumsum(sp, 0) - sp > top_p
        sp = sp.masked_fill(cut, 0)
        probs = torch.zeros_like(probs).scatter(0, si, sp)
        probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=generator))
