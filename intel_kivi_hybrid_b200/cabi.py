"""ctypes binding of libkivi_cuda.so (include/kivi_cuda.h) for torch tensors.

This is the raw C ABI: device pointers, sizes and a stream handle.  Tensors are
only used to obtain ``data_ptr()`` and the current CUDA stream.  Any non-zero
return code raises RuntimeError carrying ``kivi_last_error()``.  Importing this
module fails loudly when the library is missing and cannot be built: there is
no CPU fallback.
"""
import ctypes
import os

import torch

from . import _build

F32, BF16 = 0, 1
ROUND_HALF_AWAY, ROUND_HALF_EVEN = 0, 1
ATTN_AUTO, ATTN_FP32, ATTN_MMA = 0, 1, 2

_c = ctypes
_i64, _int, _vp, _f = _c.c_int64, _c.c_int, _c.c_void_p, _c.c_float


class Layer(_c.Structure):
    """struct kivi_layer of include/kivi_cuda.h."""
    _fields_ = [("num_units", _c.c_int32), ("head_dim", _c.c_int32), ("group_size", _c.c_int32),
                ("residual_cap", _c.c_int32), ("max_tokens", _c.c_int64), ("res_dtype", _c.c_int32),
                ("reserved", _c.c_int32), ("k_codes", _vp), ("k_scales", _vp), ("k_zeros", _vp),
                ("v_codes", _vp), ("v_scales", _vp), ("v_zeros", _vp), ("k_res", _vp), ("v_res", _vp)]


PEER_MAX_WORLD = 8


class PeerGatherDesc(_c.Structure):
    """struct kivi_peer_gather of include/kivi_cuda.h."""
    _fields_ = [("rank", _c.c_int32), ("world", _c.c_int32), ("out_ptrs", _vp * PEER_MAX_WORLD),
                ("flag_ptrs", _vp * PEER_MAX_WORLD), ("unit_offset", _c.c_int64), ("epoch", _c.c_uint32),
                ("wait", _c.c_int32), ("spin_limit", _c.c_uint32), ("reserved", _c.c_uint32), ("wait_stats", _vp),
                ("epoch_dev", _vp), ("alt_bytes", _c.c_int64)]


SIGNATURES = {
    "kivi_last_error": (_c.c_char_p, []),
    "kivi_version": (_int, []),
    "kivi_last_launch_count": (_int, []),
    "kivi_selftest_mma_alignment_bits": (_int, [_c.POINTER(_int)]),
    "kivi_device_fault": (_int, [_c.POINTER(_int)]),
    "kivi_device_fault_clear": (_int, []),
    "kivi_quantize_keys_per_channel": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _int, _int, _vp]),
    "kivi_quantize_values_per_token": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _int, _int, _int, _vp]),
    "kivi_dequantize_keys_per_channel": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _vp]),
    "kivi_dequantize_values_per_token": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _vp]),
    "kivi_quant_dequant_roundtrip_keys": (_int, [_vp, _int, _vp, _i64, _int, _int, _vp]),
    "kivi_quant_dequant_roundtrip_values": (_int, [_vp, _int, _vp, _i64, _int, _int, _int, _vp]),
    "kivi_cache_plan": (_int, [_i64, _int, _int, _int, _int, _c.POINTER(_int), _c.POINTER(_i64), _c.POINTER(_int)]),
    "kivi_cache_update": (_int, [_c.POINTER(Layer), _i64, _int, _int, _vp, _vp, _int, _i64, _i64, _i64, _i64,
                                 _int, _int, _c.POINTER(_i64), _c.POINTER(_int), _c.POINTER(_int), _vp]),
    "kivi_cache_materialize": (_int, [_c.POINTER(Layer), _i64, _int, _int, _vp, _vp, _vp]),
    "kivi_cache_import_keys": (_int, [_c.POINTER(Layer), _vp, _vp, _vp, _i64, _vp]),
    "kivi_decode_attention_workspace": (_c.c_size_t, [_int, _int, _int, _int]),
    "kivi_decode_attention_max_splits": (_int, []),
    "kivi_decode_attention_plan": (_int, [_int, _i64, _int, _int, _int, _int, _int, _int, _int, _int, _int,
                                          _c.POINTER(_int), _c.POINTER(_int), _c.POINTER(_int)]),
    "kivi_decode_attention_noalloc": (_int, [_c.POINTER(Layer), _i64, _int, _int, _vp, _int, _vp, _int, _int, _f,
                                             _int, _int, _vp]),
    "kivi_decode_attention": (_int, [_c.POINTER(Layer), _i64, _int, _int, _vp, _int, _vp, _int, _int, _f,
                                     _vp, _c.c_size_t, _int, _int, _vp]),
    "kivi_decode_attention_lse": (_int, [_c.POINTER(Layer), _i64, _int, _int, _vp, _int, _vp, _int, _vp, _int, _f,
                                         _vp, _c.c_size_t, _int, _int, _vp]),
    "kivi_decode_attention_gather": (_int, [_c.POINTER(Layer), _i64, _int, _int, _vp, _int, _c.POINTER(PeerGatherDesc),
                                            _int, _int, _f, _vp, _c.c_size_t, _int, _int, _vp]),
    "kivi_merge_token_shards": (_int, [_vp, _int, _i64, _int, _vp, _int, _vp, _vp]),
    "kivi_decode_step_stage_bytes": (_c.c_size_t, [_int, _int, _int]),
    "kivi_decode_step_host": (_int, [_c.POINTER(Layer), _c.POINTER(_i64), _c.POINTER(_int), _c.POINTER(_int),
                                     _vp, _vp, _vp, _vp, _int, _int, _int, _f, _vp, _c.c_size_t, _vp, _c.c_size_t,
                                     _int, _int, _int, _int, _int, _c.POINTER(PeerGatherDesc), _i64, _vp]),
    "kivi_sample_tokens": (_int, [_vp, _int, _int, _int, _i64, _f, _int, _int, _c.c_uint64, _c.c_uint64, _vp, _vp]),
    "kivi_peer_alloc": (_int, [_c.c_size_t, _c.POINTER(_vp), _c.c_char_p]),
    "kivi_peer_open": (_int, [_c.c_char_p, _c.POINTER(_vp)]),
    "kivi_peer_close": (_int, [_vp]),
    "kivi_peer_free": (_int, [_vp]),
}


def _load():
    path = os.environ.get("KIVI_CUDA_LIB") or _build.LIB      # override: a library built elsewhere
    if not os.path.exists(path):
        try:
            _build.build_cuda_lib()
        except Exception as exc:  # pragma: no cover - build box only
            raise ImportError(
                f"{path} is missing and could not be built with nvcc ({exc}). "
                "Run `python -m intel_kivi_hybrid_b200._build`; there is no CPU fallback.") from exc
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError = header and library out of sync
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def _check(rc):
    if rc != 0:
        raise RuntimeError(f"kivi_cuda error {rc}: {lib.kivi_last_error().decode()}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise RuntimeError(f"unsupported dtype {t.dtype}: expected float32 or bfloat16")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(*ts):
    """Every tensor of one call: on a CUDA device, contiguous, and all on the
    same device (the kernel runs on one GPU and must not be handed another
    GPU's pointers).  Raises before anything is launched."""
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("tensor must be on a CUDA device")
        if not t.is_contiguous():
            raise RuntimeError("tensor must be contiguous")
        if t.device != ts[0].device:
            raise RuntimeError(f"all tensors of one call must be on the same device, got {ts[0].device} and {t.device}")


def quantize_keys(x, packed, scales, zeros, group_size, rounding=ROUND_HALF_AWAY):
    _dev(x, packed, scales, zeros)
    _check(lib.kivi_quantize_keys_per_channel(x.data_ptr(), _dt(x), packed.data_ptr(), scales.data_ptr(),
                                              zeros.data_ptr(), scales.numel(), group_size, rounding, _stream()))


def quantize_values(x, packed, scales, zeros, head_dim, group_size, rounding=ROUND_HALF_AWAY):
    _dev(x, packed, scales, zeros)
    _check(lib.kivi_quantize_values_per_token(x.data_ptr(), _dt(x), packed.data_ptr(), scales.data_ptr(),
                                              zeros.data_ptr(), x.numel() // head_dim, head_dim, group_size,
                                              rounding, _stream()))


def dequantize_keys(packed, scales, zeros, out, group_size):
    _dev(packed, scales, zeros, out)
    _check(lib.kivi_dequantize_keys_per_channel(packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                                out.data_ptr(), scales.numel(), group_size, _stream()))


def dequantize_values(packed, scales, zeros, out, group_size):
    _dev(packed, scales, zeros, out)
    _check(lib.kivi_dequantize_values_per_token(packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                                out.data_ptr(), scales.numel(), group_size, _stream()))


def roundtrip_keys(x, out, group_size, rounding=ROUND_HALF_AWAY):
    _dev(x, out)
    _check(lib.kivi_quant_dequant_roundtrip_keys(x.data_ptr(), _dt(x), out.data_ptr(), x.numel() // group_size,
                                                 group_size, rounding, _stream()))


def roundtrip_values(x, out, head_dim, group_size, rounding=ROUND_HALF_AWAY):
    _dev(x, out)
    _check(lib.kivi_quant_dequant_roundtrip_values(x.data_ptr(), _dt(x), out.data_ptr(), x.numel() // head_dim,
                                                   head_dim, group_size, rounding, _stream()))


def mma_alignment_bits() -> int:
    """kivi_selftest_mma_alignment_bits on the current device."""
    w = _int()
    _check(lib.kivi_selftest_mma_alignment_bits(_c.byref(w)))
    return w.value


def device_fault() -> int:
    w = _int()
    _check(lib.kivi_device_fault(_c.byref(w)))
    return w.value


def device_fault_clear():
    """Reset the sticky fault word of the current device (after it was reported)."""
    _check(lib.kivi_device_fault_clear())


def cache_plan(quant_len, res_len, n_new, G, R):
    f, ql, rl = _int(), _i64(), _int()
    _check(lib.kivi_cache_plan(quant_len, res_len, n_new, G, R, _c.byref(f), _c.byref(ql), _c.byref(rl)))
    return f.value, ql.value, rl.value


def attention_plan(num_units, quant_len, res_len, head_dim=128, group_size=32, n_rep=4, q_dtype=BF16, num_splits=0,
                   path=ATTN_AUTO, sms=0, ctas_per_sm=0):
    """kivi_decode_attention_plan: (uses the tensor-core kernel, pieces per unit,
    residual-ring CTAs per unit) for a problem of this shape; sms / ctas_per_sm
    <= 0 ask the current device."""
    tc, sp, rp = _int(), _int(), _int()
    _check(lib.kivi_decode_attention_plan(num_units, quant_len, res_len, head_dim, group_size, n_rep, q_dtype,
                                          num_splits, path, sms, ctas_per_sm, _c.byref(tc), _c.byref(sp), _c.byref(rp)))
    return bool(tc.value), sp.value, rp.value


class LayerStore:
    """Device buffers of one layer + the three host counters.  Thin owner of a
    ``struct kivi_layer``; all arithmetic happens in the library."""

    def __init__(self, num_units, head_dim, group_size, residual_cap, max_tokens, dtype, device):
        G, D = group_size, head_dim
        max_tokens = -(-max_tokens // G) * G
        self.num_units, self.D, self.G, self.R, self.max_tokens = num_units, D, G, residual_cap, max_tokens
        self.dtype, self.device = dtype, torch.device(device)
        mg = max_tokens // G
        kw = dict(device=self.device)
        self.k_codes = torch.zeros(num_units, mg, D * G // 4, dtype=torch.uint8, **kw)
        self.k_scales = torch.zeros(num_units, mg, D, dtype=torch.float32, **kw)
        self.k_zeros = torch.zeros(num_units, mg, D, dtype=torch.float32, **kw)
        self.v_codes = torch.zeros(num_units, max_tokens, D // 4, dtype=torch.uint8, **kw)
        self.v_scales = torch.zeros(num_units, max_tokens, D // G, dtype=torch.float32, **kw)
        self.v_zeros = torch.zeros(num_units, max_tokens, D // G, dtype=torch.float32, **kw)
        self.k_res = torch.zeros(num_units, residual_cap, D, dtype=dtype, **kw)
        self.v_res = torch.zeros(num_units, residual_cap, D, dtype=dtype, **kw)
        self.quant_len, self.res_start, self.res_len = 0, 0, 0
        self.c = Layer(num_units, D, G, residual_cap, max_tokens, F32 if dtype == torch.float32 else BF16, 0,
                       self.k_codes.data_ptr(), self.k_scales.data_ptr(), self.k_zeros.data_ptr(),
                       self.v_codes.data_ptr(), self.v_scales.data_ptr(), self.v_zeros.data_ptr(),
                       self.k_res.data_ptr(), self.v_res.data_ptr())
        self._ws = None

    def reset(self):
        self.quant_len, self.res_start, self.res_len = 0, 0, 0

    def update(self, new_k, new_v, rounding=ROUND_HALF_AWAY):
        """new_k/new_v: [num_units, n_new, D] (a view with a unit and a token
        stride is fine as long as the last dim is contiguous)."""
        assert new_k.is_cuda and new_v.is_cuda and new_k.dtype == new_v.dtype
        assert new_k.shape == new_v.shape and new_k.shape[0] == self.num_units and new_k.shape[2] == self.D
        if new_k.stride(2) != 1:
            new_k = new_k.contiguous()
        if new_v.stride(2) != 1:
            new_v = new_v.contiguous()
        ql, rs, rl = _i64(), _int(), _int()
        _check(lib.kivi_cache_update(_c.byref(self.c), self.quant_len, self.res_start, self.res_len,
                                     new_k.data_ptr(), new_v.data_ptr(), _dt(new_k),
                                     new_k.stride(0), new_k.stride(1), new_v.stride(0), new_v.stride(1),
                                     new_k.shape[1], rounding, _c.byref(ql), _c.byref(rs), _c.byref(rl), _stream()))
        self.quant_len, self.res_start, self.res_len = ql.value, rs.value, rl.value

    def materialize(self):
        T = self.quant_len + self.res_len
        k = torch.empty(self.num_units, T, self.D, dtype=torch.float32, device=self.device)
        v = torch.empty_like(k)
        if T:
            _check(lib.kivi_cache_materialize(_c.byref(self.c), self.quant_len, self.res_start, self.res_len,
                                              k.data_ptr(), v.data_ptr(), _stream()))
        return k, v

    def import_keys(self, packed, scales, zeros, seq_len):
        _dev(packed, scales, zeros)
        _check(lib.kivi_cache_import_keys(_c.byref(self.c), packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                          seq_len, _stream()))

    def workspace(self, n_rep, num_splits=0):
        need = lib.kivi_decode_attention_workspace(self.num_units, n_rep, self.D, num_splits)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    def attention(self, q, out=None, n_rep=None, sm_scale=0.0, num_splits=0, path=ATTN_AUTO, out_dtype=None):
        """q: [num_units, n_rep, D] (or anything contiguous with that many elements)."""
        _dev(q)
        n_rep = n_rep or q.numel() // (self.num_units * self.D)
        if out is None:
            out = torch.empty(q.shape, dtype=out_dtype or q.dtype, device=q.device)
        ws = self.workspace(n_rep, num_splits)
        _check(lib.kivi_decode_attention(_c.byref(self.c), self.quant_len, self.res_start, self.res_len,
                                         q.data_ptr(), _dt(q), out.data_ptr(), _dt(out), n_rep, float(sm_scale),
                                         ws.data_ptr(), ws.numel(), num_splits, path, _stream()))
        return out

    def attention_lse(self, q, n_rep=None, sm_scale=0.0, num_splits=0, path=ATTN_AUTO, out_dtype=None, use_ring=True):
        """attention() plus the natural-log sum of exponentials per (unit, head):
        returns (out [like q], lse [num_units, n_rep] fp32).  use_ring=False
        attends to the quantized store only (a rank of a sequence-sharded cache
        that leaves the replicated ring to another rank)."""
        _dev(q)
        n_rep = n_rep or q.numel() // (self.num_units * self.D)
        out = torch.empty(q.shape, dtype=out_dtype or q.dtype, device=q.device)
        lse = torch.empty(self.num_units, n_rep, dtype=torch.float32, device=q.device)
        ws = self.workspace(n_rep, num_splits)
        _check(lib.kivi_decode_attention_lse(_c.byref(self.c), self.quant_len, self.res_start, self.res_len if use_ring else 0,
                                             q.data_ptr(), _dt(q), out.data_ptr(), _dt(out), lse.data_ptr(), n_rep,
                                             float(sm_scale), ws.data_ptr(), ws.numel(), num_splits, path, _stream()))
        return out, lse

    def attention_gather(self, q, desc: "PeerGatherDesc", out_dtype, n_rep, sm_scale=0.0, num_splits=0, path=ATTN_AUTO):
        """kivi_decode_attention_gather: the output rows of this store's units go
        straight into every rank's gathered buffer (see parallel.PeerGather)."""
        _dev(q)
        ws = self.workspace(n_rep, num_splits)
        odt = F32 if out_dtype == torch.float32 else BF16
        _check(lib.kivi_decode_attention_gather(_c.byref(self.c), self.quant_len, self.res_start, self.res_len,
                                                q.data_ptr(), _dt(q), _c.byref(desc), odt, n_rep, float(sm_scale),
                                                ws.data_ptr(), ws.numel(), num_splits, path, _stream()))

    def decode_step_host(self, h_q, h_new_k, h_new_v, h_out, n_rep, sm_scale=0.0, num_splits=0, path=ATTN_AUTO,
                         rounding=ROUND_HALF_AWAY, chunks=1, direct=True, gather=None, gather_units=0):
        """kivi_decode_step_host: one decode layer-step from pinned host tensors
        (q [units, n_rep, D], the new K and V token [units, D]) to a pinned host
        output, stream-ordered on the current stream and not synchronised; the
        store's counters advance as in update().  direct: the kernels access the
        host buffers themselves; otherwise staged copies in `chunks` runs."""
        # a decode loop passes the same four buffers every step: what was checked
        # once (is_pinned asks the driver, microseconds per tensor) is remembered
        key = (h_q.data_ptr(), h_new_k.data_ptr(), h_new_v.data_ptr(), h_out.data_ptr(), n_rep)
        if getattr(self, "_host_ok", None) != key:
            for t in (h_q, h_new_k, h_new_v, h_out):
                if t.is_cuda or not t.is_pinned() or not t.is_contiguous():
                    raise RuntimeError("decode_step_host needs contiguous pinned host tensors")
            need = lib.kivi_decode_step_stage_bytes(self.num_units, n_rep, self.D)
            if getattr(self, "_stage", None) is None or self._stage.numel() < need:
                self._stage = torch.empty(need, dtype=torch.uint8, device=self.device)
            self._host_ok = key
        ws = self.workspace(n_rep, num_splits)
        ql, rs, rl = _i64(self.quant_len), _int(self.res_start), _int(self.res_len)
        _check(lib.kivi_decode_step_host(_c.byref(self.c), _c.byref(ql), _c.byref(rs), _c.byref(rl),
                                         h_q.data_ptr(), h_new_k.data_ptr(), h_new_v.data_ptr(), h_out.data_ptr(),
                                         _dt(h_q), _dt(h_out), n_rep, float(sm_scale), self._stage.data_ptr(),
                                         self._stage.numel(), ws.data_ptr(), ws.numel(), num_splits, path, rounding,
                                         chunks, int(bool(direct)), _c.byref(gather) if gather is not None else None, gather_units,
                                         _stream()))
        self.quant_len, self.res_start, self.res_len = ql.value, rs.value, rl.value
        return h_out

    def attention_noalloc(self, q, out, n_rep, sm_scale=0.0, num_splits=0, path=ATTN_AUTO):
        """kivi_decode_attention_noalloc: same result as attention(), with the
        split partials in the library's built-in scratch array instead of a
        workspace tensor.  `out` must be preallocated by the caller: nothing is
        allocated on this path."""
        _dev(q, out)
        _check(lib.kivi_decode_attention_noalloc(_c.byref(self.c), self.quant_len, self.res_start, self.res_len,
                                                 q.data_ptr(), _dt(q), out.data_ptr(), _dt(out), n_rep,
                                                 float(sm_scale), num_splits, path, _stream()))
        return out


def merge_token_shards(parts, out_dtype=torch.float32):
    """kivi_merge_token_shards: parts [n_shards, ..., D + 1] fp32 (output rows
    followed by their log-sum-exp) -> [..., D] of out_dtype."""
    _dev(parts)
    assert parts.dtype == torch.float32 and parts.dim() >= 3
    n, D = parts.shape[0], parts.shape[-1] - 1
    rows = parts[0].numel() // (D + 1)
    out = torch.empty(parts.shape[1:-1] + (D,), dtype=out_dtype, device=parts.device)
    _check(lib.kivi_merge_token_shards(parts.data_ptr(), n, rows, D, out.data_ptr(), _dt(out), None, _stream()))
    return out


def sample_tokens(logits, temperature=1.0, top_k=0, do_sample=False, seed=0, step=0, out=None):
    """kivi_sample_tokens: [batch, vocab] fp32 / bf16 device logits (last dim
    contiguous) -> int64 [batch] device ids, without a host round trip."""
    assert logits.dim() == 2 and logits.stride(1) == 1
    if not logits.is_cuda:
        raise RuntimeError("tensor must be on a CUDA device")
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    _dev(out)
    if out.device != logits.device:
        raise RuntimeError(f"all tensors of one call must be on the same device, got {logits.device} and {out.device}")
    _check(lib.kivi_sample_tokens(logits.data_ptr(), _dt(logits), logits.shape[0], logits.shape[1], logits.stride(0),
                                  float(temperature), int(top_k or 0), int(bool(do_sample)), int(seed) & (2**64 - 1),
                                  int(step) & (2**64 - 1), out.data_ptr(), _stream()))
    return out


def quantize_groups_at(store: "LayerStore", k, v, at_group: int, rounding=ROUND_HALF_AWAY):
    """Quantize whole groups of tokens k, v [num_units, n*G, D] straight into the
    packed store of ``store`` at groups at_group .. at_group + n - 1, without
    touching its ring or counters (a view of the layer whose window is one group
    long, so every token is flushed)."""
    G = store.G
    n_tok = k.shape[1]
    assert n_tok % G == 0 and at_group * G + n_tok <= store.max_tokens
    if n_tok == 0:
        return
    shadow = Layer.from_buffer_copy(store.c)
    shadow.residual_cap = G
    ql, rs, rl = _i64(), _int(), _int()
    _check(lib.kivi_cache_update(_c.byref(shadow), at_group * G, 0, 0, k.data_ptr(), v.data_ptr(), _dt(k),
                                 k.stride(0), k.stride(1), v.stride(0), v.stride(1), n_tok, rounding,
                                 _c.byref(ql), _c.byref(rs), _c.byref(rl), _stream()))
    assert ql.value == at_group * G + n_tok and rl.value == 0


def update_discarding_flush(store: "LayerStore", scratch: "LayerStore", new_k, new_v, rounding=ROUND_HALF_AWAY):
    """store.update() for a rank that does not keep the groups this update
    flushes: the ring of ``store`` advances exactly as usual, the flushed groups
    are written to ``scratch``'s packed arrays (group 0 onwards) instead of the
    store's, and store.quant_len stays as it is."""
    shadow = Layer.from_buffer_copy(store.c)
    for name in ("k_codes", "k_scales", "k_zeros", "v_codes", "v_scales", "v_zeros"):
        setattr(shadow, name, getattr(scratch, name).data_ptr())
    shadow.max_tokens = scratch.max_tokens
    ql, rs, rl = _i64(), _int(), _int()
    _check(lib.kivi_cache_update(_c.byref(shadow), 0, store.res_start, store.res_len, new_k.data_ptr(), new_v.data_ptr(),
                                 _dt(new_k), new_k.stride(0), new_k.stride(1), new_v.stride(0), new_v.stride(1),
                                 new_k.shape[1], rounding, _c.byref(ql), _c.byref(rs), _c.byref(rl), _stream()))
    store.res_start, store.res_len = rs.value, rl.value
    return ql.value // store.G


def peer_alloc(nbytes: int):
    """(device pointer, 64-byte handle) of a zeroed allocation other processes of
    the node can map with peer_open()."""
    ptr, handle = _vp(), _c.create_string_buffer(64)
    _check(lib.kivi_peer_alloc(nbytes, _c.byref(ptr), handle))
    return ptr.value, handle.raw


def peer_open(handle: bytes) -> int:
    ptr = _vp()
    _check(lib.kivi_peer_open(_c.create_string_buffer(handle, 64), _c.byref(ptr)))
    return ptr.value


def peer_close(ptr: int):
    _check(lib.kivi_peer_close(ptr))


def peer_free(ptr: int):
    _check(lib.kivi_peer_free(ptr))


def load_state(store: "LayerStore", k_all, v_all, n_quant, rounding=ROUND_HALF_AWAY):
    """Put ``store`` into the state "first n_quant tokens quantized, the rest in
    the ring" for [num_units, T, D] device tensors.  The quantized part goes
    through kivi_cache_update on a view of the layer whose window is one group
    long (so every token is flushed); the ring is then filled directly.  Used to
    build benchmark states such as a full ring, which add_tokens never leaves
    behind (the reference flushes as soon as the window holds R tokens)."""
    G = store.G
    assert n_quant % G == 0 and k_all.shape[1] - n_quant <= store.R
    store.reset()
    if n_quant:
        shadow = Layer.from_buffer_copy(store.c)
        shadow.residual_cap = G
        ql, rs, rl = _i64(), _int(), _int()
        kq, vq = k_all[:, :n_quant], v_all[:, :n_quant]
        _check(lib.kivi_cache_update(_c.byref(shadow), 0, 0, 0, kq.data_ptr(), vq.data_ptr(), _dt(kq),
                                     kq.stride(0), kq.stride(1), vq.stride(0), vq.stride(1), n_quant, rounding,
                                     _c.byref(ql), _c.byref(rs), _c.byref(rl), _stream()))
        assert ql.value == n_quant and rl.value == 0
    n_res = k_all.shape[1] - n_quant
    if n_res:
        store.k_res[:, :n_res] = k_all[:, n_quant:].to(store.dtype)
        store.v_res[:, :n_res] = v_all[:, n_quant:].to(store.dtype)
    store.quant_len, store.res_start, store.res_len = n_quant, 0, n_res
