"""KiviCache: KIVI 2-bit asymmetric KV cache, resident on the GPU.

Drop-in for the reference's ``KiviCache`` (src/kivi_sycl/cache/manager.py:52-423):
same constructor arguments and asserts, ``from_model``, ``add_tokens``,
``get_full_cache``, ``reset``, ``get_stats``, ``total_flushes`` and the
attributes its tests read (``_quant_token_count``, ``res_keys``, ``G``, ``R``,
``num_layers``, ``batch_size``, ``num_kv_heads``).

What is different underneath: the reference keeps the residual window and a
dequantized fp32 history on the CPU and throws the packed data away
(manager.py:100-117); here every layer owns a packed store and a residual ring
in device memory (``cabi.LayerStore``), flushes run as kernels on the current
stream with no host round trip, and ``decode_attention`` attends over the
packed store directly.  ``get_full_cache`` survives as the compatibility path
for third-party model code that wants dense past_key_values.

With ``shard=(rank, world)`` a process keeps only its contiguous slice of the
(batch, kv_head) units; ``decode_attention`` then all-gathers the outputs:
``gather="nccl"`` with a collective after the kernel, ``gather="peer"`` inside
the kernel (its last stage stores every row into all ranks' buffers over
NVLink, ``parallel.PeerGather``).

With ``shard_mode="tokens"`` the *sequence* is sharded instead (fewer units than
GPUs, or one very long context): every rank holds all units and the replicated
residual ring, but only its share of each unit's quantized token groups
(``parallel.TokenShardPlan``); every rank is fed the same new tokens.
``decode_attention`` attends to the local groups (rank 0 also to the ring),
all-gathers one (output, log-sum-exp) row per query head and folds the rows
with ``kivi_merge_token_shards``.
"""
from typing import List, Optional, Tuple

import torch

from .. import cabi
from ..config.model_config import detect_model_config
from ..parallel import PeerGather, TokenShardPlan, all_gather_units, unit_partition

__all__ = ["KiviCache"]


def _iter_kv_layers(past_key_values):
    """(key, value) per layer from a legacy tuple of pairs, a Cache with
    ``.layers[i].keys/.values``, or one with ``key_cache``/``value_cache`` lists
    (same three shapes the reference accepts, manager.py:14-33)."""
    if hasattr(past_key_values, "layers"):
        for layer in past_key_values.layers:
            yield layer.keys, layer.values
    elif hasattr(past_key_values, "key_cache") and hasattr(past_key_values, "value_cache"):
        yield from zip(past_key_values.key_cache, past_key_values.value_cache)
    else:
        for item in past_key_values:
            yield item[0], item[1]


def _build_cache(layers):
    """List of (key, value) -> transformers DynamicCache through ``update``, the
    construction path that is stable across transformers versions
    (manager.py:36-49)."""
    from transformers.cache_utils import DynamicCache
    cache = DynamicCache()
    for i, (k, v) in enumerate(layers):
        cache.update(k, v, i)
    return cache


class KiviCache:
    def __init__(self, num_layers: int, head_dim: int, num_kv_heads: Optional[int] = None,
                 device: str = "cuda", group_size: int = 32, residual_length: int = 128,
                 max_tokens: int = 4096, rounding: str = "half_away",
                 shard: Optional[Tuple[int, int]] = None, gather: str = "nccl", shard_mode: str = "units"):
        assert gather in ("nccl", "peer")
        assert shard_mode in ("units", "tokens")
        assert head_dim % group_size == 0, \
            f"head_dim ({head_dim}) must be divisible by group_size ({group_size})"
        assert group_size >= 4 and group_size % 4 == 0, \
            f"group_size ({group_size}) must be >= 4 and divisible by 4"
        assert group_size <= residual_length, (
            f"group_size ({group_size}) must not exceed residual_length ({residual_length}) "
            f"- flushing requires a full group of tokens to be available in the residual buffer, "
            f"or tokens are silently dropped.")
        assert rounding in ("half_away", "half_even")
        self.device = device
        self.G = group_size
        self.R = residual_length
        self.head_dim = head_dim
        self.num_layers = num_layers
        self.num_kv_heads = num_kv_heads
        self.batch_size: Optional[int] = None
        self.rounding = cabi.ROUND_HALF_AWAY if rounding == "half_away" else cabi.ROUND_HALF_EVEN
        self.shard = shard
        self.gather = gather
        self.shard_mode = shard_mode
        # sequence sharding: the plan, the global quantized length per layer and a
        # one-group scratch store per layer for flushes another rank keeps
        self._tokens = TokenShardPlan(*shard) if (shard and shard_mode == "tokens" and shard[1] > 1) else None
        self._global_quant: List[int] = [0] * num_layers
        self._scratch: List[Optional[cabi.LayerStore]] = [None] * num_layers
        self._peer: dict = {}                              # (n_units, n_rep, dtype) -> PeerGather
        self._capacity = max(max_tokens, group_size)
        self._stores: List[Optional[cabi.LayerStore]] = [None] * num_layers
        self._flush_count: List[int] = [0] * num_layers
        self._cache_view = None
        self._cache_view_valid = False
        self._serve_device = None
        self._serve_dtype = None
        self._units: Optional[Tuple[int, int]] = None      # [u0, u1) held by this process

    @classmethod
    def from_model(cls, model, device: str = "cuda", group_size: int = 32,
                   residual_length: int = 128, **kwargs) -> "KiviCache":
        cfg = detect_model_config(model)
        return cls(num_layers=cfg["num_layers"], head_dim=cfg["head_dim"], num_kv_heads=cfg["num_kv_heads"],
                   device=device, group_size=group_size, residual_length=residual_length, **kwargs)

    # ------------------------------------------------------------------ state views
    @property
    def _quant_token_count(self) -> List[int]:
        if self._tokens is not None:             # over all ranks, not only the groups kept here
            return list(self._global_quant)
        return [0 if s is None else s.quant_len for s in self._stores]

    def _window(self, i: int, which: str) -> Optional[torch.Tensor]:
        st = self._stores[i]
        if st is None:
            return None
        ring = st.k_res if which == "k" else st.v_res
        idx = (torch.arange(st.res_len, device=ring.device) + st.res_start) % st.R
        n_local = st.num_units
        H = self.num_kv_heads
        win = ring.index_select(1, idx)
        return win.reshape(n_local // H, H, st.res_len, self.head_dim) if n_local % H == 0 else win

    @property
    def res_keys(self) -> List[Optional[torch.Tensor]]:
        """Residual window of every layer, oldest token first, [B, H, res_len, D]."""
        return [self._window(i, "k") for i in range(self.num_layers)]

    @property
    def res_values(self) -> List[Optional[torch.Tensor]]:
        return [self._window(i, "v") for i in range(self.num_layers)]

    # ------------------------------------------------------------------ core API
    def _new_store(self, n_units: int, capacity: int, dtype) -> cabi.LayerStore:
        return cabi.LayerStore(n_units, self.head_dim, self.G, self.R, capacity, dtype, self.device)

    def _ensure_capacity(self, i: int, n_new: int, dtype, n_units: int) -> cabi.LayerStore:
        st = self._stores[i]
        if st is None:
            st = self._stores[i] = self._new_store(n_units, self._capacity, dtype)
        _, need, _ = cabi.cache_plan(st.quant_len, st.res_len, n_new, self.G, self.R)
        if need > st.max_tokens:
            cap = st.max_tokens
            while cap < need:
                cap *= 2
            big = self._new_store(n_units, cap, dtype)
            ng, nt = st.quant_len // self.G, st.quant_len
            for name, n in (("k_codes", ng), ("k_scales", ng), ("k_zeros", ng),
                            ("v_codes", nt), ("v_scales", nt), ("v_zeros", nt)):
                getattr(big, name)[:, :n].copy_(getattr(st, name)[:, :n])
            big.k_res.copy_(st.k_res); big.v_res.copy_(st.v_res)
            big.quant_len, big.res_start, big.res_len = st.quant_len, st.res_start, st.res_len
            st = self._stores[i] = big
        return st

    def add_tokens(self, past_key_values):
        """Ingest the KV pairs of one forward pass (each tensor [B, H, Seq, D],
        the full cache the model returns).  Only the tokens beyond those already
        tracked are taken; they go to the residual ring and whole groups of G are
        flushed to the packed store while the window holds >= R tokens
        (manager.py:162-249)."""
        if past_key_values is not self._cache_view:
            self._cache_view_valid = False
        for i, (k, v) in enumerate(_iter_kv_layers(past_key_values)):
            self._latch_shapes(k, i)
            st = self._stores[i]
            new_start = 0
            held = 0 if st is None else (self._global_quant[i] if self._tokens is not None else st.quant_len) + st.res_len
            if held > 0:
                new_start = held
                assert k.shape[2] >= new_start, (
                    f"KiviCache desync at layer {i}: expected past length {new_start} but got {k.shape[2]}. "
                    f"add_tokens() must be called exactly once per forward pass, seeded by get_full_cache().")
            n_new = k.shape[2] - new_start
            assert n_new > 0, (
                f"KiviCache desync at layer {i}: the forward pass produced no tokens beyond the {new_start} "
                f"already tracked. add_tokens() was called twice on the same forward output, or the model was "
                f"fed a past_key_values not obtained from get_full_cache(). Silently skipping here would drop "
                f"this step's KV and corrupt all subsequent attention.")
            self.ingest_layer(i, k[:, :, new_start:, :], v[:, :, new_start:, :])

    def _latch_shapes(self, k: torch.Tensor, layer: int) -> None:
        if self.batch_size is None:
            self.batch_size = k.shape[0]
            self.num_kv_heads = k.shape[1]
            self._serve_device, self._serve_dtype = k.device, k.dtype
            n_units = self.batch_size * self.num_kv_heads
            if self.shard and self._tokens is None and self.shard[1] > 1:
                # a rank without units would never launch, and its peers would wait for it
                assert n_units >= self.shard[1], (
                    f"{n_units} (batch, kv_head) units cannot be sharded over {self.shard[1]} ranks: "
                    f"every rank must hold at least one unit")
            self._units = (unit_partition(n_units, *self.shard) if (self.shard and self._tokens is None)
                           else (0, n_units))
        else:
            assert k.shape[0] == self.batch_size, (
                f"KiviCache batch size changed mid-session ({self.batch_size} -> {k.shape[0]}) at layer {layer}. "
                f"Call reset() before starting a new request/batch.")

    def ingest_layer(self, layer: int, new_k: torch.Tensor, new_v: torch.Tensor) -> None:
        """Append the NEW tokens of one layer ([B, H, n_new, D]) to the residual
        ring and flush whole groups while the window holds >= R tokens.  This is
        the per-layer body of add_tokens(); a past_key_values object that streams
        the model's K/V into the cache calls it directly."""
        self._latch_shapes(new_k, layer)
        n_new = new_k.shape[2]
        dtype = torch.bfloat16 if new_k.dtype == torch.bfloat16 else torch.float32
        u0, u1 = self._units
        nk = new_k.flatten(0, 1)[u0:u1].to(device=self.device, dtype=dtype)
        nv = new_v.flatten(0, 1)[u0:u1].to(device=self.device, dtype=dtype)
        if self._tokens is not None:
            flushed = self._ingest_token_sharded(layer, nk, nv, dtype)
            if flushed:
                self._flush_count[layer] += flushed
            return
        st = self._ensure_capacity(layer, n_new, dtype, u1 - u0)
        before = st.quant_len
        st.update(nk, nv, self.rounding)
        flushed = (st.quant_len - before) // self.G
        if flushed:
            self._flush_count[layer] += flushed
            # flushed tokens are now served at 2-bit fidelity: the persistent
            # view no longer matches (manager.py:244-249)
            self._cache_view_valid = False

    def _ingest_token_sharded(self, layer: int, nk: torch.Tensor, nv: torch.Tensor, dtype) -> int:
        """ingest_layer() of a sequence-sharded cache: nk, nv [units, n_new, D], the
        same on every rank.  Returns the number of groups flushed (globally)."""
        G, R, plan = self.G, self.R, self._tokens
        n_units, n_new = nk.shape[0], nk.shape[1]
        st = self._stores[layer]
        if st is None:
            st = self._stores[layer] = self._new_store(n_units, self._capacity, dtype)
            self._scratch[layer] = self._new_store(n_units, 2 * G, dtype)
        res_len0 = st.res_len
        f, gq, rl = cabi.cache_plan(self._global_quant[layer], res_len0, n_new, G, R)
        if self._global_quant[layer] == 0 and res_len0 == 0 and f > 1:
            # bulk flush of an empty cache (prefill): contiguous runs of the f groups
            g0, g1 = plan.bulk_run(f)
            self._grow_token_store(layer, (g1 - g0) * G, dtype)
            st = self._stores[layer]
            cabi.quantize_groups_at(st, nk[:, g0 * G:g1 * G], nv[:, g0 * G:g1 * G], 0, self.rounding)
            st.quant_len = (g1 - g0) * G
            st.k_res[:, :rl] = nk[:, f * G:].to(st.dtype)
            st.v_res[:, :rl] = nv[:, f * G:].to(st.dtype)
            st.res_start, st.res_len = 0, rl
            self._global_quant[layer] = gq
            return f
        # otherwise feed the tokens in pieces that flush at most one group each
        flushed, t = 0, 0
        while t < n_new:
            piece = min(n_new - t, max(1, R - st.res_len))
            pk, pv = nk[:, t:t + piece], nv[:, t:t + piece]
            f1, _, _ = cabi.cache_plan(self._global_quant[layer], st.res_len, piece, G, R)
            assert f1 <= 1
            if f1 == 0 or plan.owns(self._global_quant[layer] // G):
                self._grow_token_store(layer, f1 * G, dtype)
                st = self._stores[layer]
                st.update(pk, pv, self.rounding)
            else:
                cabi.update_discarding_flush(st, self._scratch[layer], pk, pv, self.rounding)
            self._global_quant[layer] += f1 * G
            flushed += f1
            t += piece
        return flushed

    def _grow_token_store(self, layer: int, extra_tokens: int, dtype) -> None:
        """Make room for extra_tokens more locally kept quantized tokens."""
        st = self._stores[layer]
        need = st.quant_len + extra_tokens
        if need <= st.max_tokens:
            return
        cap = st.max_tokens
        while cap < need:
            cap *= 2
        big = self._new_store(st.num_units, cap, dtype)
        ng, nt = st.quant_len // self.G, st.quant_len
        for name, n in (("k_codes", ng), ("k_scales", ng), ("k_zeros", ng), ("v_codes", nt), ("v_scales", nt), ("v_zeros", nt)):
            getattr(big, name)[:, :n].copy_(getattr(st, name)[:, :n])
        big.k_res.copy_(st.k_res); big.v_res.copy_(st.v_res)
        big.quant_len, big.res_start, big.res_len = st.quant_len, st.res_start, st.res_len
        self._stores[layer] = big

    def token_shard_partial(self, layer: int, q_units: torch.Tensor, n_rep: int, num_splits: int = 0,
                            sm_scale: float = 0.0) -> torch.Tensor:
        """This rank's share of a sequence-sharded attention: [units, n_rep, D + 1]
        fp32, the output over the token groups kept here (rank 0: and the ring)
        followed by its log-sum-exp; -inf marks "no token of this row here"."""
        st = self._stores[layer]
        use_ring = self._tokens.serves_ring
        U, D = st.num_units, self.head_dim
        part = torch.empty(U, n_rep, D + 1, dtype=torch.float32, device=q_units.device)
        if st.quant_len + (st.res_len if use_ring else 0) == 0:
            part[..., :D] = 0.0
            part[..., D] = float("-inf")
            return part
        out, lse = st.attention_lse(q_units, n_rep=n_rep, out_dtype=torch.float32, num_splits=num_splits,
                                    sm_scale=sm_scale, use_ring=use_ring)
        part[..., :D] = out
        part[..., D] = lse
        return part

    def decode_attention(self, layer: int, q: torch.Tensor, out_dtype=None, num_splits: int = 0,
                         sm_scale: float = 0.0) -> torch.Tensor:
        """Fused attention of one decode step over the packed cache of ``layer``:
        softmax(q K^T / sqrt(D)) V over [quantized history || residual window].
        q: [B, Hq, D] on the cache device; returns [B, Hq, D].  No dequantized
        cache is materialised (this replaces get_full_cache + the model's own
        attention, generate.py:75-77, for callers that can hand over q).
        ``num_splits`` fixes how many pieces each unit's history is cut into
        (0 = chosen from the problem size); with the same value a sharded and an
        unsharded cache give bit-identical outputs; ``sm_scale`` overrides the
        default head_dim**-0.5."""
        st = self._stores[layer]
        assert st is not None, "decode_attention() before any add_tokens()"
        B, Hq, D = q.shape
        n_rep = Hq // self.num_kv_heads
        u0, u1 = self._units
        q_units = q.reshape(B * self.num_kv_heads, n_rep, D)[u0:u1].contiguous()
        if self._tokens is not None:
            import torch.distributed as dist
            part = self.token_shard_partial(layer, q_units, n_rep, num_splits, sm_scale)
            parts = torch.empty((self._tokens.world,) + tuple(part.shape), dtype=torch.float32, device=part.device)
            dist.all_gather_into_tensor(parts, part)
            return cabi.merge_token_shards(parts, out_dtype or q.dtype).reshape(B, Hq, D)
        if self.shard and self.shard[1] > 1 and self.gather == "peer":
            # collective on first use (buffers are exchanged once); the result is a
            # view of this rank's gathered buffer, overwritten two calls later
            key = (B * self.num_kv_heads, n_rep, out_dtype or q.dtype)
            if key not in self._peer:
                self._peer[key] = PeerGather(key[0], n_rep, D, key[2], self.shard[0], self.shard[1])
            pg = self._peer[key]
            st.attention_gather(q_units, pg.descriptor(), pg.dtype, n_rep, sm_scale=sm_scale, num_splits=num_splits)
            return pg.gathered().reshape(B, Hq, D)
        out = st.attention(q_units, n_rep=n_rep, out_dtype=out_dtype, num_splits=num_splits, sm_scale=sm_scale)
        if self.shard and self.shard[1] > 1 and self._tokens is None:
            out = all_gather_units(out, B * self.num_kv_heads, self.shard[0], self.shard[1])
        return out.reshape(B, Hq, D)

    def get_full_cache(self):
        """Dense past_key_values for unmodified model code (manager.py:251-290):
        dequantized history followed by the residual window, as a DynamicCache on
        the device and in the dtype the model handed its KV in."""
        if self._cache_view is not None and self._cache_view_valid:
            return self._cache_view
        assert not (self.shard and self.shard[1] > 1), "get_full_cache() is not available on a sharded cache"
        layers = []
        for i in range(self.num_layers):
            st = self._stores[i]
            if st is None or st.quant_len + st.res_len == 0:
                layers.append((torch.empty(0), torch.empty(0)))
                continue
            k, v = st.materialize()
            shape = (self.batch_size, self.num_kv_heads, k.shape[1], self.head_dim)
            layers.append((k.reshape(shape).to(self._serve_device, self._serve_dtype),
                           v.reshape(shape).to(self._serve_device, self._serve_dtype)))
        self._cache_view = _build_cache(layers)
        self._cache_view_valid = True
        return self._cache_view

    def check_device_fault(self) -> None:
        """Raise if a bounded wait inside one of the library's kernels has run out
        on this device since the last check: a bulk copy that never landed (bit 0,
        the affected split was dropped) or, with gather="peer", a rank that did
        not publish its rows in time (bit 1: the gathered rows of that rank were
        stale).  Reading the word synchronises the device, so this is not called
        per step; close(), reset() and state_dict() call it, and a serving loop
        should call it wherever it synchronises anyway.  The word is cleared
        before raising so the next check reports new faults only."""
        word = cabi.device_fault()
        if word:
            cabi.device_fault_clear()
            what = [name for bit, name in ((1, "a bulk copy inside the attention kernel did not land in time"),
                                           (2, "a peer rank did not publish its attention outputs in time")) if word & bit]
            raise RuntimeError("kivi_cuda device fault word = %d: %s; outputs since the last check may be wrong"
                               % (word, "; ".join(what)))

    def close(self):
        """Collective: unmap and free the peer-gather buffers (gather="peer");
        reports a peer wait that ran out since the last check."""
        for pg in self._peer.values():
            pg.close()
        self._peer = {}
        if torch.cuda.is_available():
            self.check_device_fault()

    def reset(self):
        """Clear all cached data so the same object can serve a new sequence
        (manager.py:292-303); device buffers are released and re-created lazily."""
        if any(s is not None for s in self._stores) and torch.cuda.is_available():
            self.check_device_fault()
        self._flush_count = [0] * self.num_layers
        self._stores = [None] * self.num_layers
        self._scratch = [None] * self.num_layers
        self._global_quant = [0] * self.num_layers
        self.batch_size = None
        self._cache_view = None
        self._cache_view_valid = False

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        """Everything needed to resume decoding elsewhere: per layer the packed
        store in use (codes, scales, zeros), the residual ring and the three
        counters, plus the shape bookkeeping.  Tensors are clones on the cache
        device.  (The reference has no checkpointing; its reset() is the only
        state operation, manager.py:292-303.)"""
        self.check_device_fault()
        layers = []
        for st in self._stores:
            if st is None:
                layers.append(None)
                continue
            ng, nt = st.quant_len // self.G, st.quant_len
            layers.append({
                "quant_len": st.quant_len, "res_start": st.res_start, "res_len": st.res_len,
                "num_units": st.num_units, "dtype": st.dtype,
                "k_codes": st.k_codes[:, :ng].clone(), "k_scales": st.k_scales[:, :ng].clone(),
                "k_zeros": st.k_zeros[:, :ng].clone(), "v_codes": st.v_codes[:, :nt].clone(),
                "v_scales": st.v_scales[:, :nt].clone(), "v_zeros": st.v_zeros[:, :nt].clone(),
                "k_res": st.k_res.clone(), "v_res": st.v_res.clone()})
        return {"version": 1, "G": self.G, "R": self.R, "head_dim": self.head_dim, "num_layers": self.num_layers,
                "num_kv_heads": self.num_kv_heads, "batch_size": self.batch_size, "units": self._units,
                "flush_count": list(self._flush_count), "serve_device": self._serve_device,
                "serve_dtype": self._serve_dtype, "layers": layers}

    def load_state_dict(self, state: dict) -> None:
        """Inverse of state_dict(); the cache must have been built with the same
        group_size, residual_length, head_dim and num_layers."""
        assert state["version"] == 1
        for key, mine in (("G", self.G), ("R", self.R), ("head_dim", self.head_dim), ("num_layers", self.num_layers)):
            assert state[key] == mine, f"state_dict {key}={state[key]} does not match this cache ({mine})"
        self.num_kv_heads, self.batch_size = state["num_kv_heads"], state["batch_size"]
        self._units = state["units"]
        self._flush_count = list(state["flush_count"])
        self._serve_device, self._serve_dtype = state["serve_device"], state["serve_dtype"]
        self._cache_view, self._cache_view_valid = None, False
        for i, lay in enumerate(state["layers"]):
            if lay is None:
                self._stores[i] = None
                continue
            cap = max(self._capacity, lay["quant_len"])
            st = self._new_store(lay["num_units"], cap, lay["dtype"])
            ng, nt = lay["quant_len"] // self.G, lay["quant_len"]
            for name, n in (("k_codes", ng), ("k_scales", ng), ("k_zeros", ng),
                            ("v_codes", nt), ("v_scales", nt), ("v_zeros", nt)):
                getattr(st, name)[:, :n].copy_(lay[name])
            st.k_res.copy_(lay["k_res"]); st.v_res.copy_(lay["v_res"])
            st.quant_len, st.res_start, st.res_len = lay["quant_len"], lay["res_start"], lay["res_len"]
            self._stores[i] = st

    # ------------------------------------------------------------------ stats
    @property
    def total_flushes(self) -> int:
        return sum(self._flush_count)

    def get_stats(self, layer: int = 0) -> dict:
        """Token and byte counts of one layer, same keys and formulas as the
        reference (manager.py:384-419).  ``kivi_bytes`` = packed store in use
        (codes + fp32 scales and zeros, the reference's analytic figure
        :350-356) + the residual window."""
        B = self.batch_size or 1
        H = self.num_kv_heads or 1
        st = self._stores[layer]
        D, G = self.head_dim, self.G
        quant_tokens = 0 if st is None else st.quant_len
        res_tokens = 0 if st is None else st.res_len
        total = quant_tokens + res_tokens
        per_flush = B * H * (D * (G // 4) + D * 8 + G * (D // 4) + G * (D // G) * 8)
        quant_bytes = per_flush * (quant_tokens // G)
        elem = 4 if st is None else st.k_res.element_size()
        res_bytes = 2 * B * H * res_tokens * D * elem
        fp32_bytes = 2 * B * H * total * D * 4
        kivi = quant_bytes + res_bytes
        return {"total_tokens": total, "quantized_tokens": quant_tokens, "residual_tokens": res_tokens,
                "kivi_bytes": kivi, "fp32_bytes": fp32_bytes, "compression": fp32_bytes / kivi if kivi > 0 else 0}

    def __repr__(self):
        return (f"KiviCache(layers={self.num_layers}, head_dim={self.head_dim}, "
                f"G={self.G}, R={self.R}, device='{self.device}')")
