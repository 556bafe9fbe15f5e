"""GPU tests of the drop-in Python surface: the kivi_cuda._C operators (shaped
like tests/integration/test_roundtrip_kernels.py and test_kivi.py of the
reference) and KiviCache driven the way tests/unit/test_manager_bookkeeping.py
drives the reference's cache."""
import os

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def native():
    from kivi_cuda import _C
    return _C


def test_roundtrip_keys_matches_pair_and_reference(native):
    torch.manual_seed(0)
    B, H, D, S = 2, 3, 64, 32
    x = torch.randn(B, H, D, S, device=DEV)
    fused = torch.empty_like(x)
    native.quant_dequant_roundtrip_keys(x, fused, S)
    packed = torch.empty(B, H, D, S // 4, dtype=torch.uint8, device=DEV)
    scales = torch.empty(B, H, D, device=DEV)
    zeros = torch.empty(B, H, D, device=DEV)
    native.quantize_keys(x, packed, scales, zeros, S)
    paired = torch.empty_like(x)
    native.dequantize_keys(packed, scales, zeros, paired, S)
    assert torch.equal(fused, paired)
    assert torch.allclose(fused.cpu(), ko.roundtrip_groups(x.cpu(), S), atol=1e-5) or \
        int(ko.tie_mask(x.cpu().reshape(-1, S)).sum()) > 0
    native.quant_dequant_roundtrip_keys(x, fused, S, rounding=native.ROUND_HALF_EVEN)
    assert torch.equal(fused.cpu(), ko.roundtrip_groups(x.cpu(), S))


def test_roundtrip_values_matches_pair_and_reference(native):
    torch.manual_seed(1)
    B, H, S, D, G = 2, 3, 8, 64, 32
    x = torch.randn(B, H, S, D, device=DEV)
    fused = torch.empty_like(x)
    native.quant_dequant_roundtrip_values(x, fused, D, G)
    packed = torch.empty(B, H, S, D // 4, dtype=torch.uint8, device=DEV)
    scales = torch.empty(B, H, S, D // G, device=DEV)
    zeros = torch.empty(B, H, S, D // G, device=DEV)
    native.quantize_values(input=x, output=packed, scales=scales, zeros=zeros, head_dim=D, group_size=G)
    paired = torch.empty_like(x)
    native.dequantize_values(input=packed, scales=scales, zeros=zeros, output=paired, head_dim=D, group_size=G)
    assert torch.equal(fused, paired)
    ref = ko.quantize_groups(x.cpu(), G, "half_away")
    assert torch.equal(packed.cpu().reshape(-1), ref["packed"]) and torch.equal(scales.cpu().reshape(-1), ref["scales"])


def test_known_answer_constant_and_code_range(native):
    x = torch.tensor([[[[1.0, 2.0, 3.0, 4.0]]]], device=DEV)
    packed = torch.empty(1, 1, 1, 1, dtype=torch.uint8, device=DEV)
    scales = torch.empty(1, 1, 1, device=DEV)
    zeros = torch.empty(1, 1, 1, device=DEV)
    native.quantize_keys(x, packed, scales, zeros, 4)
    assert packed.item() == 228 and abs(scales.item() - 1.0) < 0.01 and abs(zeros.item() - 1.0) < 0.01
    out = torch.empty_like(x)
    native.dequantize_keys(packed, scales, zeros, out, 4)
    assert (out.cpu().squeeze() - torch.tensor([1.0, 2.0, 3.0, 4.0])).abs().max() < 0.1
    c = torch.full((1, 1, 4, 32), 5.0, device=DEV)
    o = torch.empty_like(c)
    native.quant_dequant_roundtrip_keys(c, o, 32)
    assert torch.isfinite(o).all() and torch.allclose(o, c, atol=1e-4)
    # error bound and code range of test_kivi.py:53-90
    k = torch.randn(1, 2, 4, 32, device=DEV)
    p = torch.empty(1, 2, 4, 8, dtype=torch.uint8, device=DEV)
    s = torch.empty(1, 2, 4, device=DEV)
    z = torch.empty(1, 2, 4, device=DEV)
    native.quantize_keys(k, p, s, z, 32)
    d = torch.empty_like(k)
    native.dequantize_keys(p, s, z, d, 32)
    assert (d - k).abs().max() <= 0.6 * s.max()
    assert int(ko.unpack_codes(p.cpu()).max()) <= 3


def test_async_ops_and_event(native):
    x = torch.randn(4, 8, 128, 64, device=DEV)
    out = torch.full_like(x, float("nan"))
    ev = native.quant_dequant_roundtrip_values_async(x, out, 64, 32)
    assert isinstance(ev, native.KiviEvent)
    ev.wait()
    assert torch.equal(out.cpu(), ko.roundtrip_groups(x.cpu(), 32, "half_away"))
    packed = torch.empty(x.numel() // 4, dtype=torch.uint8, device=DEV)
    scales = torch.empty(x.numel() // 32, device=DEV)
    zeros = torch.empty_like(scales)
    e1 = native.quantize_keys_async(x, packed, scales, zeros, 32)
    back = torch.empty_like(x)
    e2 = native.dequantize_keys_async(packed, scales, zeros, back, 32)    # same stream: ordered behind e1
    e2.wait(); e1.wait()
    assert torch.equal(back, out)
    # bf16 input is accepted (upcast in registers) and equals quantizing its fp32 upcast
    xb = x.to(torch.bfloat16)
    native.quant_dequant_roundtrip_keys(xb, out, 32)
    assert torch.equal(out.cpu(), ko.roundtrip_groups(xb.float().cpu(), 32, "half_away"))


def test_operator_validation_messages(native):
    x = torch.randn(64, device=DEV)
    p = torch.empty(16, dtype=torch.uint8, device=DEV)
    s = torch.empty(2, device=DEV)
    z = torch.empty(2, device=DEV)
    with pytest.raises(RuntimeError, match="divisible by 4"):
        native.quantize_keys(x, p, s, z, 6)
    with pytest.raises(RuntimeError, match="must equal num_channels"):
        native.quantize_keys(x, p, s, z, 16)
    with pytest.raises(RuntimeError, match="zeros size"):
        native.quantize_keys(x, p, s, torch.empty(3, device=DEV), 32)
    with pytest.raises(RuntimeError, match="refusing to silently truncate"):
        native.quantize_values(x, p, s, z, 48, 16)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        native.quant_dequant_roundtrip_keys(torch.randn(8, 16, device=DEV).t(), torch.empty(16, 8, device=DEV), 8)
    with pytest.raises(RuntimeError, match="must be Byte"):
        native.dequantize_keys(x, s, z, x, 32)
    with pytest.raises(RuntimeError, match="shape-preserving"):
        native.quant_dequant_roundtrip_keys(x, torch.empty(32, device=DEV), 32)


# ---- KiviCache ----------------------------------------------------------------

class FakeModel:
    """Stands in for a HuggingFace forward pass: token t of every layer is filled
    with the value t (+ small noise) so a dropped or reordered token shows up;
    ``in_place`` grows the DynamicCache it is handed, ``legacy_tuple`` returns
    fresh full-length tuples (the two KV contracts the reference tests)."""

    def __init__(self, layers, heads, dim, mode, device="cpu"):
        self.L, self.H, self.D, self.mode, self.device = layers, heads, dim, mode, device
        self.total = 0
        self.truth_k = [None] * layers
        self.truth_v = [None] * layers
        self.gen = torch.Generator().manual_seed(99)

    def forward(self, n_new, past=None):
        from transformers.cache_utils import DynamicCache
        from intel_kivi_hybrid_b200.cache.manager import _iter_kv_layers
        new = []
        for i in range(self.L):
            base = torch.arange(self.total, self.total + n_new, dtype=torch.float32).view(1, 1, n_new, 1)
            base = base.expand(1, self.H, n_new, self.D)
            jit = torch.randn(1, self.H, n_new, self.D, generator=self.gen) * 0.01
            k, v = (base + jit).contiguous().to(self.device), (base - jit).contiguous().to(self.device)
            new.append((k, v))
            self.truth_k[i] = k if self.truth_k[i] is None else torch.cat([self.truth_k[i], k], 2)
            self.truth_v[i] = v if self.truth_v[i] is None else torch.cat([self.truth_v[i], v], 2)
        past_t = None
        if past is not None:
            past_t = list(_iter_kv_layers(past))
            for pk, _ in past_t:
                assert pk.shape[2] == self.total, f"served {pk.shape[2]} past tokens, expected {self.total}"
        self.total += n_new
        if self.mode == "in_place":
            cache = past if isinstance(past, DynamicCache) else DynamicCache()
            for i, (k, v) in enumerate(new):
                cache.update(k, v, i)
            return cache
        out = []
        for i, (k, v) in enumerate(new):
            if past_t is not None:
                k, v = torch.cat([past_t[i][0], k], 2), torch.cat([past_t[i][1], v], 2)
            out.append((k, v))
        return tuple(out)


@pytest.mark.parametrize("mode", ["in_place", "legacy_tuple"])
@pytest.mark.parametrize("model_device", ["cpu", "cuda"])
def test_flushed_history_matches_kivi_reference(mode, model_device):
    from kivi_sycl import KiviCache
    from intel_kivi_hybrid_b200.cache.manager import _iter_kv_layers
    G, R, D, L, H = 4, 8, 8, 2, 2
    cache = KiviCache(num_layers=L, head_dim=D, num_kv_heads=H, device=DEV, group_size=G, residual_length=R,
                      rounding="half_even")
    model = FakeModel(L, H, D, mode, model_device)
    cache.add_tokens(model.forward(6))
    for _ in range(24):
        past = cache.get_full_cache()
        served = next(iter(_iter_kv_layers(past)))[0].shape[2]
        assert served == model.total, "stale cache served: generated tokens are being dropped"
        cache.add_tokens(model.forward(1, past))
    for i, (k, v) in enumerate(_iter_kv_layers(cache.get_full_cache())):
        n_hist = cache._quant_token_count[i]
        assert n_hist > 0 and k.shape[2] == model.total
        assert torch.equal(k[:, :, n_hist:].cpu(), model.truth_k[i][:, :, n_hist:].cpu())     # residual exact
        assert torch.equal(cache.res_keys[i].cpu(), model.truth_k[i][:, :, n_hist:].cpu())
        for c0 in range(0, n_hist, G):                                                        # history: per flush chunk
            ck = model.truth_k[i][:, :, c0:c0 + G].cpu().transpose(2, 3).contiguous()
            assert torch.equal(k[:, :, c0:c0 + G].cpu(), ko.roundtrip_groups(ck, G).transpose(2, 3))
            cv = model.truth_v[i][:, :, c0:c0 + G].cpu().contiguous()
            assert torch.equal(v[:, :, c0:c0 + G].cpu(), ko.roundtrip_groups(cv, G))
    assert cache.total_flushes == L * (cache._quant_token_count[0] // G)


def test_double_add_tokens_fails_loudly():
    from kivi_sycl import KiviCache
    cache = KiviCache(num_layers=1, head_dim=8, num_kv_heads=2, device=DEV, group_size=4, residual_length=8)
    model = FakeModel(1, 2, 8, "in_place")
    out = model.forward(5)
    cache.add_tokens(out)
    with pytest.raises(AssertionError, match="desync"):
        cache.add_tokens(out)
    cache.reset()
    assert cache.batch_size is None and cache._quant_token_count == [0]
    cache.add_tokens(out)                                   # usable again after reset()


def test_long_run_matches_reference_cache_and_stats(golden_dir):
    from kivi_sycl import KiviCache
    from intel_kivi_hybrid_b200.cache.manager import _iter_kv_layers
    sm = np.load(os.path.join(golden_dir, "state_machine_vectors.npz"))
    K, V = torch.from_numpy(sm["long__K"]), torch.from_numpy(sm["long__V"])
    cache = KiviCache(num_layers=1, head_dim=64, num_kv_heads=3, device=DEV, group_size=32, residual_length=128,
                      max_tokens=64, rounding="half_even")        # small capacity: exercises growth
    cache.add_tokens(((K[:, :, :200], V[:, :, :200]),))
    for t in range(200, 300):
        cache.add_tokens(((K[:, :, :t + 1], V[:, :, :t + 1]),))
    k, v = next(iter(_iter_kv_layers(cache.get_full_cache())))
    assert torch.equal(k, torch.from_numpy(sm["long__served_k"])) and torch.equal(v, torch.from_numpy(sm["long__served_v"]))
    assert cache.total_flushes == int(sm["long__total_flushes"])
    st = cache.get_stats(0)
    for key in ("total_tokens", "quantized_tokens", "residual_tokens", "kivi_bytes", "fp32_bytes"):
        assert st[key] == int(sm[f"long__stat_{key}"]), key
    assert abs(st["compression"] - float(sm["long__stat_compression"])) < 1e-9


def test_decode_attention_through_kivicache():
    from kivi_sycl import KiviCache
    B, Hkv, n_rep, D, T = 2, 4, 4, 128, 700
    K = ko.make_keys(B, Hkv, T, D, 31).to(torch.bfloat16)
    V = ko.make_values(B, Hkv, T, D, 31).to(torch.bfloat16)
    q = ko.make_queries(B, Hkv * n_rep, D, 31).to(torch.bfloat16)
    cache = KiviCache(num_layers=2, head_dim=D, device=DEV)
    cache.add_tokens(((K[:, :, :T - 1].cuda(), V[:, :, :T - 1].cuda()),) * 2)
    cache.add_tokens(((K.cuda(), V.cuda()),) * 2)
    n_quant = cache._quant_token_count[1]
    assert n_quant == ko.flush_schedule(*ko.flush_schedule(0, 0, T - 1, 32, 128)[1:], 1, 32, 128)[1]
    out = cache.decode_attention(1, q.cuda(), out_dtype=torch.float32)
    ref = ko.kivi_decode_attention(q, K, V, n_quant, 32, "half_away", dtype=torch.float64).float()
    err = ((out.cpu() - ref).abs().amax(-1) / ref.abs().amax(-1)).max().item()
    assert out.shape == (B, Hkv * n_rep, D) and err < 2e-3


def test_state_dict_round_trip_resumes_bit_identically():
    from kivi_sycl import KiviCache
    B, Hkv, n_rep, D, T = 1, 2, 4, 128, 420
    K = ko.make_keys(B, Hkv, T, D, 9).to(torch.bfloat16).cuda()
    V = ko.make_values(B, Hkv, T, D, 9).to(torch.bfloat16).cuda()
    q = ko.make_queries(B, Hkv * n_rep, D, 9).to(torch.bfloat16).cuda()
    a = KiviCache(num_layers=1, head_dim=D, device=DEV)
    a.add_tokens(((K[:, :, :300], V[:, :, :300]),))
    state = a.state_dict()
    b = KiviCache(num_layers=1, head_dim=D, device=DEV)
    b.load_state_dict(state)
    for c in (a, b):                                      # both continue with the same tokens
        for t in range(300, T):
            c.add_tokens(((K[:, :, :t + 1], V[:, :, :t + 1]),))
    assert a._quant_token_count == b._quant_token_count and a.total_flushes == b.total_flushes
    assert torch.equal(a.decode_attention(0, q), b.decode_attention(0, q))
    assert a.get_stats() == b.get_stats()


@pytest.mark.parametrize("dtype,D,G,n_rep", [(torch.bfloat16, 128, 32, 4), (torch.float32, 64, 32, 1)])
def test_cache_operators_of_the_extension(native, dtype, D, G, n_rep):
    """_C.append_and_flush + _C.decode_attention on caller-owned tensors: same
    counters and bit-identical stores / outputs as the ctypes path over the same
    library, and the attention within tolerance of the oracle."""
    from intel_kivi_hybrid_b200 import cabi
    B, H, R, T, cap = 1, 3, 128, 333, 512
    U = B * H
    K = ko.make_keys(B, H, T, D, seed=31)
    V = ko.make_values(B, H, T, D, seed=31)
    q = ko.make_queries(B, H * n_rep, D, seed=31)
    if dtype == torch.bfloat16:
        K, V, q = K.bfloat16().float(), V.bfloat16().float(), q.bfloat16().float()
    kc = K.reshape(U, T, D).to(DEV, dtype)
    vc = V.reshape(U, T, D).to(DEV, dtype)
    mg = cap // G
    t = dict(k_packed=torch.zeros(U, mg, D * G // 4, dtype=torch.uint8, device=DEV),
             k_scales=torch.zeros(U, mg, D, device=DEV), k_zeros=torch.zeros(U, mg, D, device=DEV),
             v_packed=torch.zeros(U, cap, D // 4, dtype=torch.uint8, device=DEV),
             v_scales=torch.zeros(U, cap, D // G, device=DEV), v_zeros=torch.zeros(U, cap, D // G, device=DEV),
             k_res=torch.zeros(U, R, D, dtype=dtype, device=DEV), v_res=torch.zeros(U, R, D, dtype=dtype, device=DEV))
    st = cabi.LayerStore(U, D, G, R, cap, dtype, DEV)
    state = (0, 0, 0)
    for a, b in ((0, 200), (200, 201), (201, T)):
        state = native.append_and_flush(kc[:, a:b], vc[:, a:b], quant_len=state[0], res_start=state[1], res_len=state[2],
                                        group_size=G, **t)
        st.update(kc[:, a:b], vc[:, a:b])
        assert tuple(state) == (st.quant_len, st.res_start, st.res_len)
    for name in t:
        assert torch.equal(t[name], getattr(st, {"k_packed": "k_codes", "v_packed": "v_codes"}.get(name, name))), name
    qd = q.reshape(U, n_rep, D).to(DEV, dtype)
    out = torch.full((U, n_rep, D), float("nan"), device=DEV, dtype=torch.float32)
    native.decode_attention(qd, quant_len=state[0], res_start=state[1], res_len=state[2], out=out, group_size=G, **t)
    ws = torch.empty(native.decode_attention_workspace(U, n_rep, D), dtype=torch.uint8, device=DEV)
    out2 = torch.empty_like(out)
    native.decode_attention(qd, t["k_packed"], t["k_scales"], t["k_zeros"], t["v_packed"], t["v_scales"], t["v_zeros"],
                            t["k_res"], t["v_res"], state[0], state[1], state[2], out2, G, workspace=ws)
    ref_out = st.attention(qd, n_rep=n_rep, out_dtype=torch.float32)
    assert torch.equal(out, ref_out) and torch.equal(out2, ref_out)
    oracle = ko.kivi_decode_attention(q, K, V, state[0], G, "half_away", dtype=torch.float64).float().reshape(U, n_rep, D)
    err = float(((out.cpu() - oracle).abs().amax(-1) / oracle.abs().amax(-1)).max())
    assert err < (2e-3 if dtype == torch.bfloat16 else 1e-5), err
    # validation: numel relations and dtypes, raised before anything is launched
    with pytest.raises(RuntimeError, match="k_packed size"):
        native.decode_attention(qd, t["k_packed"][:, :-1].contiguous(), t["k_scales"], t["k_zeros"], t["v_packed"], t["v_scales"],
                                t["v_zeros"], t["k_res"], t["v_res"], state[0], state[1], state[2], out, G)
    with pytest.raises(RuntimeError, match="must be on cuda"):
        native.decode_attention(qd.cpu(), quant_len=state[0], res_start=state[1], res_len=state[2], out=out, group_size=G, **t)
    with pytest.raises(RuntimeError, match="n_new, head_dim"):
        native.append_and_flush(kc[:, :4, : D // 2], vc[:, :4, : D // 2], quant_len=state[0], res_start=state[1],
                                res_len=state[2], group_size=G, **t)


def test_reference_flush_sequence_over_the_extension_reproduces_its_served_cache(native, golden_dir):
    """What the reference's own KiviCache does with its native module, replayed
    call for call over kivi_cuda._C: keep the window as a tensor, and while it
    holds >= R tokens take the oldest G, round-trip the transposed key chunk
    [B,H,D,G] and the value chunk [B,H,G,D] through the fused operators and
    append them to the history (cache/manager.py:226-243, 332-363).  The served
    history || window must equal what the reference's KiviCache served for the
    same token stream (golden vectors made by running it)."""
    sm = np.load(os.path.join(golden_dir, "state_machine_vectors.npz"))
    K, V = torch.from_numpy(sm["long__K"]).to(DEV), torch.from_numpy(sm["long__V"]).to(DEV)
    G, R, D = 32, 128, 64
    mode = native.ROUND_HALF_EVEN                          # the golden run used the reference's torch mirror
    hist_k, hist_v = [], []
    res_k, res_v = K[:, :, :0], V[:, :, :0]
    flushes = 0

    def add(k_new, v_new):
        nonlocal res_k, res_v, flushes
        res_k, res_v = torch.cat([res_k, k_new], dim=2), torch.cat([res_v, v_new], dim=2)
        while res_k.shape[2] >= R:
            ck = res_k[:, :, :G].transpose(2, 3).contiguous()           # [B,H,D,G]
            cv = res_v[:, :, :G].contiguous()                            # [B,H,G,D]
            ok, ov = torch.empty_like(ck), torch.empty_like(cv)
            native.quant_dequant_roundtrip_keys(ck, ok, G, rounding=mode)
            native.quant_dequant_roundtrip_values(cv, ov, D, G, rounding=mode)
            hist_k.append(ok.transpose(2, 3)); hist_v.append(ov)
            res_k, res_v = res_k[:, :, G:], res_v[:, :, G:]
            flushes += 1

    add(K[:, :, :200], V[:, :, :200])
    for t in range(200, 300):
        add(K[:, :, t:t + 1], V[:, :, t:t + 1])
    served_k, served_v = torch.cat(hist_k + [res_k], dim=2), torch.cat(hist_v + [res_v], dim=2)
    assert flushes == int(sm["long__total_flushes"])
    assert torch.equal(served_k.cpu(), torch.from_numpy(sm["long__served_k"]))
    assert torch.equal(served_v.cpu(), torch.from_numpy(sm["long__served_v"]))
