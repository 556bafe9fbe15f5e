"""Next-token choice for the generate() loop (reference:
src/kivi_sycl/generation/sampling.py:10-25): argmax unless ``do_sample``;
otherwise temperature scaling, optional top-k cut, softmax, one multinomial
draw.  Returns ids of shape [batch, 1]."""
from typing import Optional

import torch

__all__ = ["sample_token"]


def sample_token(logits: torch.Tensor, temperature: float, top_k: Optional[int], do_sample: bool) -> torch.Tensor:
    if not do_sample:
        return torch.argmax(logits, dim=-1, keepdim=True)
    scaled = logits / max(temperature, 1e-8)
    if top_k is not None:
        kth = torch.topk(scaled, top_k, dim=-1).values[:, -1:]
        scaled = scaled.masked_fill(scaled < kth, float("-inf"))
    return torch.multinomial(torch.softmax(scaled, dim=-1), num_samples=1)
