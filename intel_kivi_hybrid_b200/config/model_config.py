"""KV-cache shape discovery from a HuggingFace-style ``model.config``.

Same contract as the reference's detect_model_config
(src/kivi_sycl/config/model_config.py:6-59): returns ``num_layers``,
``num_kv_heads`` (KV heads, which differ from query heads under grouped-query
attention) and ``head_dim``, trying the attribute names the common model
families use and raising ValueError with a hint when one cannot be found.
"""

__all__ = ["detect_model_config"]

_LAYER_ATTRS = ("n_layer", "num_hidden_layers", "num_layers", "n_layers")
_KV_HEAD_ATTRS = ("num_key_value_heads", "num_kv_heads")
_Q_HEAD_ATTRS = ("n_head", "num_attention_heads", "num_heads")
_HIDDEN_ATTRS = ("hidden_size", "n_embd")


def _first(config, names):
    for name in names:
        if hasattr(config, name):
            return getattr(config, name)
    return None


def detect_model_config(model) -> dict:
    config = model.config
    kind = type(config).__name__

    num_layers = _first(config, _LAYER_ATTRS)
    if num_layers is None:
        raise ValueError(f"Cannot detect num_layers from {kind}. Pass num_layers= explicitly.")

    num_kv_heads = _first(config, _KV_HEAD_ATTRS)
    if num_kv_heads is None:
        num_kv_heads = _first(config, _Q_HEAD_ATTRS)
    if num_kv_heads is None:
        raise ValueError(f"Cannot detect num_heads from {kind}. Pass num_kv_heads= explicitly.")

    head_dim = getattr(config, "head_dim", None) if hasattr(config, "head_dim") else None
    if head_dim is None:
        hidden = _first(config, _HIDDEN_ATTRS)
        q_heads = _first(config, ("num_attention_heads", "n_head"))
        if not hidden or not q_heads:
            raise ValueError(f"Cannot detect head_dim from {kind}. Pass head_dim= explicitly.")
        head_dim = hidden // q_heads

    return {"num_layers": num_layers, "num_kv_heads": num_kv_heads, "head_dim": head_dim}
