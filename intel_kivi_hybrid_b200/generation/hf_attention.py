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
  Any other pattern (several query tokens on a non-empty cache, a padded decode
  batch, sliding-window layers) raises instead of attending to the wrong keys.

One ordering difference from the reference loop: ``update()`` appends the step's
token and flushes *before* the step attends, so on a flush step (one in G) the
oldest G tokens are already attended at 2-bit fidelity, one step earlier than in
generate.py:75-77, where the model attends first and add_tokens() flushes after.

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


def _mask_hides_something(attention_mask) -> bool:
    """True if an attention mask excludes any key position (costs a device sync:
    only evaluated for batched decode steps, where padding can occur)."""
    if attention_mask is None:
        return False
    if attention_mask.dtype == torch.bool:
        return not bool(attention_mask.all())
    return bool((attention_mask != 0).any())


def kivi_fused_attention(module, query, key, value, attention_mask, dropout=0.0, scaling=None, **kwargs):
    """query [B, Hq, Lq, D]; key/value: the NEW tokens of this forward pass.

    Supported call patterns: one forward over the whole prompt on an empty cache,
    then forwards of one token each -- the loop of generate().  Everything else
    would silently attend to the wrong keys and is refused: several query tokens
    on a cache that already holds a history (chunked prefill, a second chat turn,
    speculative tokens), a decode step whose mask hides positions (left-padded
    batches), and sliding-window layers.
    """
    cache = getattr(module, "_kivi_cache", None)
    B, Hq, Lq, D = query.shape
    layer = getattr(module, "layer_idx", None)
    if cache is None or layer is None:
        out = torch.nn.functional.scaled_dot_product_attention(
            query, key, value, is_causal=Lq > 1, scale=scaling, enable_gqa=key.shape[1] != Hq)
        return out.transpose(1, 2).contiguous(), None
    store = cache._stores[layer]
    held = 0 if store is None else store.quant_len + store.res_len      # includes this pass's tokens (update() ran)
    history = held - key.shape[2]
    window = kwargs.get("sliding_window", None) or getattr(module, "sliding_window", None)
    if window is not None and held > int(window):
        raise RuntimeError(f"kivi_fused attention: layer {layer} uses a sliding window of {window} tokens but the cache "
                           f"holds {held}; windowed layers are not supported by the fused decode kernel")
    if Lq == 1 and history > 0:
        if B > 1 and _mask_hides_something(attention_mask):
            raise RuntimeError("kivi_fused attention: the decode step's attention_mask hides key positions (padded batch); "
                               "the fused kernel attends to every cached token. Use get_full_cache() for padded batches.")
        q = query[:, :, 0].to(cache.device)
        if q.dtype not in (torch.float32, torch.bfloat16):
            q = q.float()
        out = cache.decode_attention(layer, q.contiguous(), sm_scale=float(scaling or 0.0))
        return out.to(query.device, query.dtype).reshape(B, 1, Hq, D), None
    if history > 0:
        raise RuntimeError(f"kivi_fused attention: {Lq} query tokens on a cache that already holds {history} tokens "
                           f"(chunked prefill / multi-token step) is not supported: the packed history would be ignored. "
                           f"Feed the prompt in one forward pass, or use get_full_cache() for this step.")
    # prefill on an empty cache: attention over the prompt's own K/V, under the
    # model's mask when it built one (padding), plain causal otherwise
    gqa = key.shape[1] != Hq
    if attention_mask is not None and attention_mask.dim() == 4 and attention_mask.shape[-1] == key.shape[2]:
        out = torch.nn.functional.scaled_dot_product_attention(query, key, value, attn_mask=attention_mask,
                                                               scale=scaling, enable_gqa=gqa)
    else:
        out = torch.nn.functional.scaled_dot_product_attention(query, key, value, is_causal=Lq > 1,
                                                               scale=scaling, enable_gqa=gqa)
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
