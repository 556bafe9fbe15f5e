"""generate(): greedy / sampled decoding of a HuggingFace CausalLM with the KV
cache held in KIVI 2-bit form on the GPU.

Same signature and loop as the reference (src/kivi_sycl/generation/generate.py:
13-89): prefill, ingest the model's past_key_values, then per step serve the
cache, run the model on the last token, ingest, pick the next token; stop at
EOS.  The model's forward (third-party code) stays wherever the caller put the
model; only the cache lives on ``device``.

The reference reads every new id back (``next_id.item()``, generate.py:72) to
test it against EOS, one host synchronisation per token.  Here the id is chosen
on the device (``sampling.sample_token``) and stays there; EOS is looked for
once every ``EOS_CHECK_EVERY`` steps over the ids produced since the last look,
and what was generated past the first EOS is cut off, so the returned text is
the same and at most ``EOS_CHECK_EVERY - 1`` steps are spent in vain.
"""
from typing import Optional

import torch

from ..cache.manager import KiviCache
from .sampling import sample_token

__all__ = ["generate"]

EOS_CHECK_EVERY = 8


def _first_eos(produced, start, eos_id):
    """Index of the first EOS among produced[start:], or None (one device->host read)."""
    if eos_id is None or start >= len(produced):
        return None
    hit = (torch.cat(produced[start:], dim=1)[0] == eos_id).nonzero()
    return start + int(hit[0, 0]) if hit.numel() else None


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
    checked = 0
    for step in range(1, max_new_tokens):
        if eos_id is not None and (step - 1) % EOS_CHECK_EVERY == 0:
            stop = _first_eos(produced, checked, eos_id)
            checked = len(produced)
            if stop is not None:
                del produced[stop + 1:]
                break
        out = model(next_id, past_key_values=cache.get_full_cache(), use_cache=True)
        cache.add_tokens(out.past_key_values)
        next_id = sample_token(out.logits[:, -1, :], temperature, top_k, do_sample).to(model_device)
        produced.append(next_id)
        if verbose and (step + 1) % 10 == 0:
            print(".", end="", flush=True)
    stop = _first_eos(produced, checked, eos_id)
    if stop is not None:
        del produced[stop + 1:]
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
        checked = 0
        for step in range(1, max_new_tokens):
            if eos_id is not None and (step - 1) % EOS_CHECK_EVERY == 0:
                stop = _first_eos(produced, checked, eos_id)
                checked = len(produced)
                if stop is not None:
                    del produced[stop + 1:]
                    break
            out = model(next_id, past_key_values=past, use_cache=True)
            next_id = sample_token(out.logits[:, -1, :], temperature, top_k, do_sample).to(model_device)
            produced.append(next_id)
            if verbose and (step + 1) % 10 == 0:
                print(".", end="", flush=True)
        stop = _first_eos(produced, checked, eos_id)
        if stop is not None:
            del produced[stop + 1:]
    if verbose:
        print()
    full = torch.cat([input_ids, torch.cat(produced, dim=1)], dim=1)
    return tokenizer.decode(full[0], skip_special_tokens=True)
