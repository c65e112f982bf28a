"""Token selection from a step's logits.  Greedy arg-max is what the reference's evaluation uses (generate(..., do_sample=False),
evaluations/models/llava_multiimg_siglip_anyres.py:448-452); temperature / top-k sampling is offered for the language models.
Selection runs on the device; only the chosen ids come back to the host (the stopping criterion needs them)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.0       # 0: greedy
    top_k: int = 0                 # 0: the whole vocabulary
    seed: Optional[int] = None


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None):
        self.p = params or SamplingParams()
        self._gen = None

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        """logits fp32 [n, vocab] -> ids int64 [n] (on the logits' device)."""
        p = self.p
        if p.temperature <= 0.0:
            return logits.argmax(-1)
        if self._gen is None:
            self._gen = torch.Generator(device=logits.device)
            if p.seed is not None:
                self._gen.manual_seed(p.seed)
        z = logits / p.temperature
        if p.top_k > 0 and p.top_k < z.shape[-1]:
            kth = z.topk(p.top_k, -1).values[:, -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        return torch.multinomial(torch.softmax(z, -1), 1, generator=self._gen).squeeze(-1)
