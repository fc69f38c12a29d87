"""Next-token sampling on the device: greedy, temperature, top-k and nucleus (top-p) filtering.  Logits are fp32 [rows, vocab]."""
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.0        # 0 = greedy
    top_k: int = 0                  # 0 = off
    top_p: float = 1.0              # 1 = off
    seed: Optional[int] = None


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None, device=None):
        self.p = params or SamplingParams()
        self.gen = None
        if self.p.seed is not None and device is not None:
            self.gen = torch.Generator(device=device).manual_seed(self.p.seed)

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        """[rows, vocab] -> [rows] int64 token ids."""
        p = self.p
        if p.temperature <= 0.0:
            return torch.argmax(logits, dim=-1)
        z = logits / p.temperature
        if p.top_k > 0:
            kth = torch.topk(z, min(p.top_k, z.shape[-1]), dim=-1).values[:, -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        if p.top_p < 1.0:
            sz, idx = torch.sort(z, dim=-1, descending=True)
            cum = torch.cumsum(torch.softmax(sz, dim=-1), dim=-1)
            drop = cum - torch.softmax(sz, dim=-1) >= p.top_p          # keep the smallest prefix whose mass reaches top_p
            sz = sz.masked_fill(drop, float("-inf"))
            z = torch.full_like(z, float("-inf")).scatter(-1, idx, sz)
        probs = torch.softmax(z, dim=-1)
        return torch.multinomial(probs, 1, generator=self.gen).squeeze(-1)
