"""Fused-attention hook for HuggingFace models.

The reference serves a dense fp32 cache to the model and lets the model's own
attention run over it (generation/generate.py:75-77, cache/manager.py:251-290).
With this hook the model never sees a dense history:

* ``KiviPastKeyValues`` is the ``past_key_values`` object handed to the model.
  Its ``update()`` streams the layer's new K/V straight into the KiviCache
  (ring append + flush on the GPU) and returns only those new tokens.
* ``kivi_fused`` is an attention function registered with transformers'
  ``AttentionInterface``.  For a decode step (one query token) it calls
  ``KiviCache.decode_attention`` -- the fused kernel over packed codes + ring;
  for the prefill (many query tokens, empty cache) it runs ordinary causal
  attention over the prompt's own K/V, exactly what the reference's prefill
  forward computes before the cache sees the tokens (generate.py:61-62).

``attached(model, cache)`` switches the model to that attention function for
the duration of a ``with`` block and restores it afterwards.
"""
import contextlib

import torch
from transformers.cache_utils import DynamicCache

__all__ = ["KiviPastKeyValues", "attached", "ATTN_NAME"]

ATTN_NAME = "kivi_fused"


class KiviPastKeyValues(DynamicCache):
    """Cache object for the model side of the hook: keeps no tensors itself."""

    def __init__(self, kivi_cache):
        super().__init__()
        self.kivi = kivi_cache
        self._seen = [0] * kivi_cache.num_layers

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.kivi.ingest_layer(layer_idx, key_states, value_states)
        self._seen[layer_idx] += key_states.shape[2]
        return key_states, value_states

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen[layer_idx]

    def get_mask_sizes(self, query_length, layer_idx: int = 0):
        # (kv_length, kv_offset) for the mask builder; transformers passes the query
        # length as an int (older releases: the cache_position tensor).  Only the
        # prefill is attended through a mask, the decode step ignores it.
        q_len = int(query_length) if isinstance(query_length, int) else int(query_length.shape[0])
        return q_len + self._seen[layer_idx], 0

    @property
    def is_compileable(self) -> bool:
        return False


def kivi_fused_attention(module, query, key, value, attention_mask, dropout=0.0, scaling=None, **kwargs):
    """query [B, Hq, Lq, D]; key/value: the NEW tokens of this forward pass."""
    cache = getattr(module, "_kivi_cache", None)
    B, Hq, Lq, D = query.shape
    layer = getattr(module, "layer_idx", None)
    if cache is not None and layer is not None and Lq == 1 and cache._quant_token_count[layer] + \
            (cache._stores[layer].res_len if cache._stores[layer] is not None else 0) > key.shape[2]:
        q = query[:, :, 0].to(cache.device)
        if q.dtype not in (torch.float32, torch.bfloat16):
            q = q.float()
        out = cache.decode_attention(layer, q.contiguous(), sm_scale=float(scaling or 0.0))
        return out.to(query.device, query.dtype).reshape(B, 1, Hq, D), None
    # prefill (or a model without a cache attached): causal attention over the new tokens
    out = torch.nn.functional.scaled_dot_product_attention(
        query, key, value, is_causal=Lq > 1, scale=scaling, enable_gqa=key.shape[1] != Hq)
    return out.transpose(1, 2).contiguous(), None


def _register():
    from transformers.masking_utils import AttentionMaskInterface, sdpa_mask
    from transformers.modeling_utils import AttentionInterface
    AttentionInterface.register(ATTN_NAME, kivi_fused_attention)
    AttentionMaskInterface.register(ATTN_NAME, sdpa_mask)


@contextlib.contextmanager
def attached(model, kivi_cache):
    """Route ``model``'s self-attention through the KIVI cache; yields the
    past_key_values object to pass to the model."""
    _register()
    previous = model.config._attn_implementation
    touched = []
    for mod in model.modules():
        if hasattr(mod, "layer_idx") and hasattr(mod, "forward") and not hasattr(mod, "_kivi_cache"):
            mod._kivi_cache = kivi_cache
            touched.append(mod)
    model.config._attn_implementation = ATTN_NAME
    try:
        yield KiviPastKeyValues(kivi_cache)
    finally:
        model.config._attn_implementation = previous
        for mod in touched:
            del mod._kivi_cache
