"""Next-token choice for the generate() loop (reference:
src/kivi_sycl/generation/sampling.py:10-25): argmax unless ``do_sample``;
otherwise temperature scaling, optional top-k cut, softmax, one multinomial
draw.  Returns ids of shape [batch, 1].

Logits that live on a CUDA device are handled by one kernel of the library
(``kivi_sample_tokens``): the ids stay on the device, so the decode loop needs no
host round trip per token.  Its draws come from a counter-based generator whose
key is taken, call by call, from torch's default CPU generator (so
``torch.manual_seed`` makes a run repeatable, as it does for the reference's
``torch.multinomial``, and drawing the key touches no device).  Logits on the
CPU (a model kept on the host, as in the reference's own set-up) go through the
same torch operations the reference uses.
"""
from typing import Optional

import torch

__all__ = ["sample_token", "DeviceSampler"]


class DeviceSampler:
    """(seed, step) bookkeeping of the device-side draws.  With a fixed ``seed``
    every call advances ``step``; without one, each sampling call draws a fresh
    62-bit key from torch's default CPU generator."""

    def __init__(self, seed: Optional[int] = None):
        self.seed = None if seed is None else int(seed)
        self.step = 0

    def __call__(self, logits: torch.Tensor, temperature: float, top_k: Optional[int], do_sample: bool) -> torch.Tensor:
        from .. import cabi
        if logits.dtype not in (torch.float32, torch.bfloat16):
            logits = logits.float()
        if logits.stride(-1) != 1:
            logits = logits.contiguous()
        if self.seed is None:       # a fresh key per call: the counter stays at 0
            seed, step = (int(torch.randint(0, 2 ** 62, (1,)).item()) if do_sample else 0), 0
        else:
            seed, step = self.seed, self.step
            self.step += 1
        return cabi.sample_tokens(logits, temperature, top_k or 0, do_sample, seed, step).unsqueeze(1)


_default = None


def sample_token(logits: torch.Tensor, temperature: float, top_k: Optional[int], do_sample: bool) -> torch.Tensor:
    global _default
    if logits.is_cuda:
        if _default is None:
            _default = DeviceSampler()
        return _default(logits, temperature, top_k, do_sample)
    if not do_sample:
        return torch.argmax(logits, dim=-1, keepdim=True)
    scaled = logits / max(temperature, 1e-8)
    if top_k is not None:
        kth = torch.topk(scaled, top_k, dim=-1).values[:, -1:]
        scaled = scaled.masked_fill(scaled < kth, float("-inf"))
    return torch.multinomial(torch.softmax(scaled, dim=-1), num_samples=1)
