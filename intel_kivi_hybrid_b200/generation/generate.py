"""generate(): greedy / sampled decoding of a HuggingFace CausalLM with the KV
cache held in KIVI 2-bit form on the GPU.

Same signature and loop as the reference (src/kivi_sycl/generation/generate.py:
13-89): prefill, ingest the model's past_key_values, then per step serve the
cache, run the model on the last token, ingest, pick the next token; stop at
EOS.  The model's forward (third-party code) stays wherever the caller put the
model; only the cache lives on ``device``.
"""
from typing import Optional

import torch

from ..cache.manager import KiviCache
from .sampling import sample_token

__all__ = ["generate"]


@torch.no_grad()
def generate(model, tokenizer, prompt: str, max_new_tokens: int = 200, group_size: int = 32,
             residual_length: int = 128, device: str = "cuda", temperature: float = 1.0,
             top_k: Optional[int] = None, do_sample: bool = False, verbose: bool = False,
             fused_attention: bool = False) -> str:
    if fused_attention:
        return _generate_fused(model, tokenizer, prompt, max_new_tokens, group_size, residual_length, device,
                               temperature, top_k, do_sample, verbose)
    cache = KiviCache.from_model(model, device=device, group_size=group_size, residual_length=residual_length)
    input_ids = tokenizer(prompt, return_tensors="pt").input_ids
    model_device = next(model.parameters()).device if hasattr(model, "parameters") else input_ids.device
    input_ids = input_ids.to(model_device)

    out = model(input_ids, use_cache=True)                                   # prefill
    cache.add_tokens(out.past_key_values)
    next_id = sample_token(out.logits[:, -1, :], temperature, top_k, do_sample)
    produced = [next_id]
    eos_id = tokenizer.eos_token_id

    # the prefill already produced token 1, so max_new_tokens - 1 more steps
    for step in range(1, max_new_tokens):
        if eos_id is not None and next_id.item() == eos_id:
            break
        out = model(next_id, past_key_values=cache.get_full_cache(), use_cache=True)
        cache.add_tokens(out.past_key_values)
        next_id = sample_token(out.logits[:, -1, :], temperature, top_k, do_sample)
        produced.append(next_id)
        if verbose and (step + 1) % 10 == 0:
            print(".", end="", flush=True)
    if verbose:
        print()
    full = torch.cat([input_ids, torch.cat(produced, dim=1)], dim=1)
    return tokenizer.decode(full[0], skip_special_tokens=True)


def _generate_fused(model, tokenizer, prompt, max_new_tokens, group_size, residual_length, device,
                    temperature, top_k, do_sample, verbose) -> str:
    """Same loop with ``fused_attention=True``: the model's K/V stream straight
    into the cache and every decode step attends through
    ``KiviCache.decode_attention`` (no dense past_key_values is ever built)."""
    from .hf_attention import attached
    cache = KiviCache.from_model(model, device=device, group_size=group_size, residual_length=residual_length)
    input_ids = tokenizer(prompt, return_tensors="pt").input_ids
    model_device = next(model.parameters()).device if hasattr(model, "parameters") else input_ids.device
    input_ids = input_ids.to(model_device)
    eos_id = tokenizer.eos_token_id
    with attached(model, cache) as past:
        out = model(input_ids, past_key_values=past, use_cache=True)
        next_id = sample_token(out.logits[:, -1, :], temperature, top_k, do_sample)
        produced = [next_id]
        for step in range(1, max_new_tokens):
            if eos_id is not None and next_id.item() == eos_id:
                break
            out = model(next_id, past_key_values=past, use_cache=True)
            next_id = sample_token(out.logits[:, -1, :], temperature, top_k, do_sample)
            produced.append(next_id)
            if verbose and (step + 1) % 10 == 0:
                print(".", end="", flush=True)
    if verbose:
        print()
    full = torch.cat([input_ids, torch.cat(produced, dim=1)], dim=1)
    return tokenizer.decode(full[0], skip_special_tokens=True)
