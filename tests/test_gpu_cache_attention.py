"""GPU parity of the device-resident cache and the fused decode attention,
through the C ABI, against the oracle and the reference-made golden vectors.

Tolerances: fp32 activations 1e-5; bf16 activations 2e-3, on the error of a
(unit, head) output row relative to the row's largest reference element,
max|out-ref| / max|ref| (`rel_err`).  The tests also print the element-wise
figure max |out-ref| / max(|ref|, 1e-3 * max|ref| of the row) (`elem_err`),
which weighs the same absolute error against each element's own magnitude."""
import os

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_BF16 = 2e-3


@pytest.fixture(scope="module")
def cabi():
    from intel_kivi_hybrid_b200 import cabi as m
    return m


def rel_err(out, ref):
    out, ref = out.float().cpu(), ref.float().cpu()
    num = (out - ref).abs().amax(dim=-1)
    den = ref.abs().amax(dim=-1).clamp_min(1e-30)
    return float((num / den).max())


def elem_err(out, ref):
    out, ref = out.float().cpu(), ref.float().cpu()
    floor = 1e-3 * ref.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((out - ref).abs() / torch.maximum(ref.abs(), floor)).max())


def units(x):            # [B,H,T,D] -> [B*H,T,D]
    return x.reshape(x.shape[0] * x.shape[1], *x.shape[2:])


def test_state_machine_matches_reference_cache(cabi, golden_dir):
    sm = np.load(os.path.join(golden_dir, "state_machine_vectors.npz"))
    K, V = torch.from_numpy(sm["long__K"]), torch.from_numpy(sm["long__V"])
    st = cabi.LayerStore(3, 64, 32, 128, 512, torch.float32, "cuda")
    Kc, Vc = units(K).cuda(), units(V).cuda()
    st.update(Kc[:, :200], Vc[:, :200], cabi.ROUND_HALF_EVEN)
    assert (st.quant_len, st.res_len) == (96, 104)
    for t in range(200, 300):
        st.update(Kc[:, t:t + 1], Vc[:, t:t + 1], cabi.ROUND_HALF_EVEN)
    assert st.quant_len == int(sm["long__quant_tokens"])
    k, v = st.materialize()
    assert torch.equal(k.cpu().reshape(1, 3, -1, 64), torch.from_numpy(sm["long__served_k"]))
    assert torch.equal(v.cpu().reshape(1, 3, -1, 64), torch.from_numpy(sm["long__served_v"]))


def test_small_g_state_machine_matches_reference_cache(cabi, golden_dir):
    sm = np.load(os.path.join(golden_dir, "state_machine_vectors.npz"))
    steps, prefill, G, R, D, layers, heads = [int(v) for v in sm["params"]]
    for i in range(layers):
        truth = torch.from_numpy(sm[f"in_place__truth_k{i}"])
        tk = units(truth).cuda()
        tv = (2 * torch.arange(truth.shape[2]).view(1, 1, -1, 1).float() - truth)
        tv = units(tv).cuda()
        st = cabi.LayerStore(heads, D, G, R, 64, torch.float32, "cuda")
        st.update(tk[:, :prefill], tv[:, :prefill], cabi.ROUND_HALF_EVEN)
        for t in range(prefill, prefill + steps):
            st.update(tk[:, t:t + 1], tv[:, t:t + 1], cabi.ROUND_HALF_EVEN)
        k, _ = st.materialize()
        assert torch.equal(k.cpu().reshape(1, heads, -1, D), torch.from_numpy(sm[f"in_place__served_k{i}"]))
        assert st.quant_len == int(sm["in_place__quant_tokens"][i])


def test_packed_store_matches_oracle_flush_by_flush(cabi):
    B, H, D, G, R = 1, 4, 64, 32, 128
    K = ko.make_keys(B, H, 300, D, seed=21)
    V = ko.make_values(B, H, 300, D, seed=21)
    oc = ko.OracleCache(D, G, R, rounding="half_away")
    st = cabi.LayerStore(B * H, D, G, R, 512, torch.float32, "cuda")
    Kc, Vc = units(K).cuda(), units(V).cuda()
    oc.append(K[:, :, :150], V[:, :, :150]); st.update(Kc[:, :150], Vc[:, :150])
    for t in range(150, 300):
        oc.append(K[:, :, t:t + 1], V[:, :, t:t + 1]); st.update(Kc[:, t:t + 1], Vc[:, t:t + 1])
    assert st.quant_len == oc.quantized_len and st.res_len == oc.residual_len
    ng = st.quant_len // G
    ks = torch.stack(oc.k_scales, dim=2).reshape(B * H, ng, D)
    kz = torch.stack(oc.k_zeros, dim=2).reshape(B * H, ng, D)
    assert torch.equal(st.k_scales[:, :ng].cpu(), ks) and torch.equal(st.k_zeros[:, :ng].cpu(), kz)
    vs = torch.cat(oc.v_scales, dim=2).reshape(B * H, ng * G, D // G)
    assert torch.equal(st.v_scales[:, :ng * G].cpu(), vs)
    vp = torch.cat(oc.v_packed, dim=2).reshape(B * H, ng * G, D // 4)
    assert torch.equal(st.v_codes[:, :ng * G].cpu(), vp)
    # key blocks hold the same codes as the reference layout, re-laid out
    kc = ko.unpack_codes(torch.stack(oc.k_packed, dim=2).reshape(B * H, ng, D, G // 4))   # [u,g,D,G]
    blk = st.k_codes[:, :ng].cpu().reshape(B * H, ng, G // 4, D)                            # one 64-wide half: [j][p(d)]
    perm = torch.tensor([(d & 3) | (((d >> 4) & 3) << 2) | (((d >> 2) & 3) << 4) for d in range(D)])
    blk = blk[..., perm]                                                                    # -> [j][d]
    Q = G // 4
    for e in range(4):
        got = (blk >> (2 * e)) & 3                       # bit pair e of byte j = token 4j + e
        assert torch.equal(got.transpose(2, 3), kc[..., e::4].to(torch.uint8))
    # served tensors: history round trip + exact residual
    k, v = st.materialize()
    sk, sv = oc.served()
    assert torch.equal(k.cpu(), units(sk)) and torch.equal(v.cpu(), units(sv))


def test_value_blocks_of_llama_shaped_layers_hold_the_reference_bytes(cabi):
    """D=128, G=32 layers store each 32-token value group as a re-laid block;
    undoing the documented permutation must give the reference's packed rows, and
    the served tensors must equal the oracle's bit for bit."""
    B, H, D, G, R = 1, 2, 128, 32, 128
    K = ko.make_keys(B, H, 200, D, seed=8)
    V = ko.make_values(B, H, 200, D, seed=8)
    oc = ko.OracleCache(D, G, R, rounding="half_away")
    st = cabi.LayerStore(B * H, D, G, R, 256, torch.float32, "cuda")
    oc.append(K, V); st.update(units(K).cuda(), units(V).cuda())
    ng = st.quant_len // G
    assert ng == oc.flushes == 3
    vp = torch.cat(oc.v_packed, dim=2).reshape(B * H, ng, G, D // 4)               # natural rows [t][b]
    blk = st.v_codes[:, :ng * G].cpu().reshape(B * H, ng, 4, 2, 8, 4, 4)            # [gd][kappa][r][c][n]
    nat = blk.permute(0, 1, 3, 5, 6, 2, 4).reshape(B * H, ng, G, D // 4)            # t = 16k+4c+n, b = 8gd+r
    assert torch.equal(nat, vp)
    vs = torch.cat(oc.v_scales, dim=2).reshape(B * H, ng, G, D // G)
    rows = st.v_scales[:, :ng * G].cpu().reshape(B * H, ng, 2, 4, 4, D // G)        # [kappa][n][c]
    assert torch.equal(rows.permute(0, 1, 2, 4, 3, 5).reshape(B * H, ng, G, D // G), vs)
    k, v = st.materialize()
    sk, sv = oc.served()
    assert torch.equal(k.cpu(), units(sk)) and torch.equal(v.cpu(), units(sv))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding", ["half_away", "half_even"])
def test_chunked_bulk_prefill_mixes_ring_and_new_tensor_groups(cabi, dtype, rounding):
    """Bulk updates whose first groups still hold ring tokens (virtual-sequence
    kernels) and whose remaining groups are cut straight out of the new tensor
    (direct kernels), in ragged chunks; one key channel and one value group carry
    a range so large that the scale has no reciprocal (plain-division branch)."""
    B, H, D, G, R = 1, 3, 128, 32, 128
    chunks = [50, 333, 1, 700, 95]
    T = sum(chunks)
    K = ko.make_keys(B, H, T, D, seed=5)
    V = ko.make_values(B, H, T, D, seed=6)
    K[0, 1, 400:420, 7] = 1.6e38; K[0, 1, 420:440, 7] = -1.6e38
    V[0, 2, 500, 32:48] = 1.6e38; V[0, 2, 500, 48:64] = -1.6e38
    if dtype == torch.bfloat16:
        K, V = K.bfloat16().float(), V.bfloat16().float()
    oc = ko.OracleCache(D, G, R, rounding=rounding)
    st = cabi.LayerStore(B * H, D, G, R, 1184, dtype, "cuda")
    mode = cabi.ROUND_HALF_EVEN if rounding == "half_even" else cabi.ROUND_HALF_AWAY
    Kc, Vc = units(K).cuda().to(dtype), units(V).cuda().to(dtype)
    t = 0
    for n in chunks:
        oc.append(K[:, :, t:t + n], V[:, :, t:t + n])
        st.update(Kc[:, t:t + n], Vc[:, t:t + n], mode)
        t += n
        assert st.quant_len == oc.quantized_len and st.res_len == oc.residual_len
    ng = st.quant_len // G
    ks = torch.stack(oc.k_scales, dim=2).reshape(B * H, ng, D)
    kz = torch.stack(oc.k_zeros, dim=2).reshape(B * H, ng, D)
    assert torch.equal(st.k_scales[:, :ng].cpu(), ks) and torch.equal(st.k_zeros[:, :ng].cpu(), kz)
    assert float(ks.max()) >= 1e30
    k, v = st.materialize()
    sk, sv = oc.served()
    assert torch.equal(k.cpu(), units(sk)) and torch.equal(v.cpu(), units(sv))


def test_import_keys_from_operator_layout(cabi):
    B, H, D, G, S = 1, 2, 128, 32, 96
    K = ko.make_keys(B, H, S, D, seed=3)
    kt = units(K).transpose(1, 2).contiguous().cuda()          # [u, D, S]
    packed = torch.empty(B * H, D, S // 4, dtype=torch.uint8, device="cuda")
    scales = torch.empty(B * H, D, S // G, device="cuda")
    zeros = torch.empty(B * H, D, S // G, device="cuda")
    cabi.quantize_keys(kt, packed, scales, zeros, G)
    a = cabi.LayerStore(B * H, D, G, 128, S, torch.float32, "cuda")
    a.import_keys(packed, scales, zeros, S)
    b = cabi.LayerStore(B * H, D, G, 128, S, torch.float32, "cuda")
    cabi.load_state(b, units(K).cuda(), units(K).cuda(), S)
    assert torch.equal(a.k_codes, b.k_codes) and torch.equal(a.k_scales, b.k_scales) and torch.equal(a.k_zeros, b.k_zeros)


def _attention_case(cabi, B, Hkv, n_rep, D, G, R, n_quant, n_res, dtype, seed, path, num_splits=0,
                    res_start=0, out_dtype=torch.float32):
    T = n_quant + n_res
    K = ko.make_keys(B, Hkv, T, D, seed).to(dtype)
    V = ko.make_values(B, Hkv, T, D, seed).to(dtype)
    q = ko.make_queries(B, Hkv * n_rep, D, seed).to(dtype)
    ref = ko.kivi_decode_attention(q, K, V, n_quant, G, "half_away")
    ref64 = ko.kivi_decode_attention(q, K, V, n_quant, G, "half_away", dtype=torch.float64)
    st = cabi.LayerStore(B * Hkv, D, G, R, max(n_quant, G), dtype, "cuda")
    cabi.load_state(st, units(K).cuda(), units(V).cuda(), n_quant)
    if res_start:                       # rotate the ring: same window, different slots
        st.k_res.copy_(torch.roll(st.k_res, res_start, dims=1))
        st.v_res.copy_(torch.roll(st.v_res, res_start, dims=1))
        st.res_start = res_start % R
    out = st.attention(q.cuda().contiguous(), n_rep=n_rep, num_splits=num_splits, path=path, out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    return rel_err(out, ref64.float()), rel_err(ref, ref64.float()), out, ref64


def test_attention_golden_seed42(cabi, golden_dir):
    av = np.load(os.path.join(golden_dir, "attention_vectors.npz"))
    q, k, v = (torch.from_numpy(av[n]) for n in ("query", "key", "value"))
    st = cabi.LayerStore(2, 64, 32, 128, 32, torch.float32, "cuda")
    cabi.load_state(st, units(k).cuda(), units(v).cuda(), 32, cabi.ROUND_HALF_EVEN)
    for i in range(q.shape[2]):
        out = st.attention(q[:, :, i].contiguous().cuda(), n_rep=1)
        assert rel_err(out, torch.from_numpy(av["out_kivi"])[:, :, i]) < TOL_F32


@pytest.mark.parametrize("n_quant,n_res,res_start", [(416, 96, 0), (608, 104, 40), (0, 77, 0), (96, 0, 0), (32, 1, 127)])
def test_attention_fp32_gpt2_shapes(cabi, n_quant, n_res, res_start):
    # config 0: B=1, H=12 (MHA), D=64, fp32, R=128, G=32
    err, oerr, _, _ = _attention_case(cabi, 1, 12, 1, 64, 32, 128, n_quant, n_res, torch.float32, 7,
                                      cabi.ATTN_FP32, res_start=res_start)
    print(f"[attn fp32 cfg0 q={n_quant} r={n_res}] rel err {err:.2e} (fp32 oracle vs fp64: {oerr:.2e})")
    assert err < TOL_F32


@pytest.mark.parametrize("D,G,n_rep", [(128, 32, 4), (128, 64, 2), (64, 16, 1), (128, 128, 8), (256, 32, 2), (32, 4, 3)])
def test_attention_fp32_shapes(cabi, D, G, n_rep):
    err, _, _, _ = _attention_case(cabi, 2, 2, n_rep, D, G, max(G, 64), 4 * G, max(G, 64) - 3, torch.float32, 11,
                                   cabi.ATTN_FP32)
    assert err < TOL_F32


@pytest.mark.parametrize("splits", [1, 2, 7, 31])
def test_attention_split_count_does_not_change_result(cabi, splits):
    err, _, out, _ = _attention_case(cabi, 1, 2, 4, 128, 32, 128, 31 * 32, 128, torch.float32, 5,
                                     cabi.ATTN_FP32, num_splits=splits)
    assert err < TOL_F32


@pytest.mark.parametrize("path,dtype,splits", [("fp32", torch.float32, 40), ("fp32", torch.float32, 100),
                                               ("mma", torch.bfloat16, 33), ("mma", torch.bfloat16, 70)])
def test_attention_with_more_than_32_partials_per_unit(cabi, path, dtype, splits):
    """The merge walks a row's partials 32 at a time, eight loads in flight: more
    than 32 pieces per unit (few units, long context) take its second round."""
    kernel = cabi.ATTN_FP32 if path == "fp32" else cabi.ATTN_MMA
    err, _, out, _ = _attention_case(cabi, 1, 2, 4, 128, 32, 128, 100 * 32, 128, dtype, 23, kernel, num_splits=splits)
    assert err < (TOL_F32 if dtype == torch.float32 else TOL_BF16)
    assert cabi.device_fault() == 0


def test_attention_bf16_llama_shape_fp32_kernel(cabi):
    # config 1 slice: GQA 4:1, D=128, bf16 activations, full ring
    err, _, _, _ = _attention_case(cabi, 2, 8, 4, 128, 32, 128, 3968, 128, torch.bfloat16, 13, cabi.ATTN_FP32)
    print(f"[attn bf16 cfg1 slice, fp32 kernel] rel err {err:.2e}")
    assert err < TOL_BF16
    err, _, _, _ = _attention_case(cabi, 2, 8, 4, 128, 32, 128, 3968, 128, torch.bfloat16, 13, cabi.ATTN_FP32,
                                   out_dtype=torch.bfloat16)
    assert err < 2 * TOL_BF16          # + half an ulp of the bf16 output itself


def test_attention_errors(cabi):
    st = cabi.LayerStore(2, 64, 32, 128, 64, torch.float32, "cuda")
    q = torch.randn(2, 1, 64, device="cuda")
    with pytest.raises(RuntimeError, match="empty"):
        st.attention(q)
    with pytest.raises(RuntimeError, match="no new tokens"):
        st.update(torch.empty(2, 0, 64, device="cuda"), torch.empty(2, 0, 64, device="cuda"))
    with pytest.raises(RuntimeError, match="overflow"):
        st.update(torch.randn(2, 400, 64, device="cuda"), torch.randn(2, 400, 64, device="cuda"))


# ---- tensor-core kernel ------------------------------------------------------

@pytest.mark.parametrize("n_quant,n_res,n_rep,splits", [
    (3968, 128, 4, 0), (32, 0, 4, 0), (64, 5, 4, 1), (96, 128, 4, 3), (2048 + 32, 100, 4, 5),
    (992, 128, 1, 0), (992, 128, 2, 2), (992, 128, 3, 0), (13 * 32, 96, 4, 13),
    (992, 128, 8, 0), (2048 + 32, 100, 5, 3), (96, 7, 6, 1), (64, 0, 7, 0)])
def test_attention_mma_bf16(cabi, n_quant, n_res, n_rep, splits):
    err, _, out, ref64 = _attention_case(cabi, 2, 4, n_rep, 128, 32, 128, n_quant, n_res, torch.bfloat16, 17,
                                         cabi.ATTN_MMA, num_splits=splits)
    print(f"[attn mma bf16 q={n_quant} r={n_res} rep={n_rep} splits={splits}] rel err {err:.2e}, "
          f"element-wise {elem_err(out, ref64.float()):.2e}")
    assert err < TOL_BF16
    assert cabi.device_fault() == 0


def test_attention_mma_matches_fp32_kernel_and_auto_dispatch(cabi):
    e_mma, _, o_mma, _ = _attention_case(cabi, 2, 8, 4, 128, 32, 128, 3968, 128, torch.bfloat16, 13, cabi.ATTN_MMA)
    e_auto, _, o_auto, _ = _attention_case(cabi, 2, 8, 4, 128, 32, 128, 3968, 128, torch.bfloat16, 13, cabi.ATTN_AUTO)
    e_f32, _, o_f32, _ = _attention_case(cabi, 2, 8, 4, 128, 32, 128, 3968, 128, torch.bfloat16, 13, cabi.ATTN_FP32)
    assert torch.equal(o_mma, o_auto)                 # bf16 queries dispatch to the tensor-core kernel
    _, _, _, ref64 = _attention_case(cabi, 2, 8, 4, 128, 32, 128, 3968, 128, torch.bfloat16, 13, cabi.ATTN_FP32)
    print(f"[attn cfg1 slice] mma {e_mma:.2e}  fp32 kernel {e_f32:.2e}  mma vs fp32 kernel {rel_err(o_mma, o_f32):.2e}; "
          f"element-wise: mma {elem_err(o_mma, ref64.float()):.2e}  fp32 kernel {elem_err(o_f32, ref64.float()):.2e}")
    assert e_mma < TOL_BF16 and rel_err(o_mma, o_f32) < TOL_BF16


def test_attention_mma_fp32_queries_and_bf16_output(cabi):
    err, _, _, _ = _attention_case(cabi, 1, 4, 4, 128, 32, 128, 1024, 64, torch.float32, 23, cabi.ATTN_MMA)
    print(f"[attn mma fp32 activations] rel err {err:.2e}")
    assert err < TOL_BF16
    err, _, _, _ = _attention_case(cabi, 1, 4, 4, 128, 32, 128, 1024, 64, torch.bfloat16, 23, cabi.ATTN_MMA,
                                   out_dtype=torch.bfloat16)
    assert err < 2 * TOL_BF16


def test_attention_mma_is_deterministic(cabi):
    _, _, a, _ = _attention_case(cabi, 2, 4, 4, 128, 32, 128, 2048, 128, torch.bfloat16, 3, cabi.ATTN_MMA)
    _, _, b, _ = _attention_case(cabi, 2, 4, 4, 128, 32, 128, 2048, 128, torch.bfloat16, 3, cabi.ATTN_MMA)
    assert torch.equal(a, b)


def test_attention_mma_rejects_other_shapes(cabi):
    st = cabi.LayerStore(2, 64, 32, 128, 64, torch.float32, "cuda")
    cabi.load_state(st, torch.randn(2, 64, 64, device="cuda"), torch.randn(2, 64, 64, device="cuda"), 64)
    with pytest.raises(RuntimeError, match="tensor-core path"):
        st.attention(torch.randn(2, 1, 64, device="cuda"), path=cabi.ATTN_MMA)


# ---- full-size properties (config 2 of the benchmark: 512 units x 32768 tokens) ----

def test_full_size_config2_properties(cabi):
    """At the benchmark's full size the oracle is too slow, so check properties that
    do not depend on size: the result does not depend on the number of splits, the
    tensor-core and the fp32 kernel agree, every output is a convex combination of
    value rows (inside their per-channel range), and a slice of units reproduces
    the CPU oracle."""
    B, Hkv, n_rep, D, G, R, n_quant, n_res = 64, 8, 4, 128, 32, 128, 32640, 128
    U, T = B * Hkv, n_quant + n_res
    g = torch.Generator(device="cuda").manual_seed(123)
    k = torch.empty(U, T, D, device="cuda", dtype=torch.bfloat16)
    v = torch.empty(U, T, D, device="cuda", dtype=torch.bfloat16)
    for u0 in range(0, U, 64):
        k[u0:u0 + 64] = torch.randn(64, T, D, device="cuda", generator=g).to(torch.bfloat16)
        v[u0:u0 + 64] = torch.randn(64, T, D, device="cuda", generator=g).to(torch.bfloat16)
    k[:, :, 5] *= 10.0                                     # an outlier channel
    st = cabi.LayerStore(U, D, G, R, n_quant, torch.bfloat16, "cuda")
    cabi.load_state(st, k, v, n_quant)
    q = torch.randn(U, n_rep, D, device="cuda", generator=g).to(torch.bfloat16)
    o_auto = st.attention(q, n_rep=n_rep, path=cabi.ATTN_MMA, out_dtype=torch.float32)
    o_s1 = st.attention(q, n_rep=n_rep, path=cabi.ATTN_MMA, num_splits=1, out_dtype=torch.float32)
    o_s9 = st.attention(q, n_rep=n_rep, path=cabi.ATTN_MMA, num_splits=9, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert cabi.device_fault() == 0 and torch.isfinite(o_auto).all()
    # different split counts change the running max that p = 2^(s-m) is taken against, hence the
    # fp16 rounding of p*s: agreement is at the level of that rounding, not bitwise
    e1, e9 = rel_err(o_s1, o_auto), rel_err(o_s9, o_auto)
    print(f"[cfg2 full size] splits 1 vs auto {e1:.2e}, 9 vs auto {e9:.2e}")
    assert e1 < TOL_BF16 and e9 < TOL_BF16
    # fp32 kernel on the last units (a full run of it takes ~5 ms; slicing needs a second store)
    sub = slice(U - 8, U)
    st8 = cabi.LayerStore(8, D, G, R, n_quant, torch.bfloat16, "cuda")
    cabi.load_state(st8, k[sub], v[sub], n_quant)
    o_f32 = st8.attention(q[sub].contiguous(), n_rep=n_rep, path=cabi.ATTN_FP32, out_dtype=torch.float32)
    print(f"[cfg2 full size] tensor-core vs fp32 kernel {rel_err(o_auto[sub], o_f32):.2e}")
    assert rel_err(o_auto[sub], o_f32) < TOL_BF16
    # convexity: the quantized values stay inside [min, max] of their group, so the output
    # stays inside the per-channel range of the unit's values
    vmin = v.float().amin(dim=1, keepdim=True)
    vmax = v.float().amax(dim=1, keepdim=True)
    eps = 1e-2
    assert bool(((o_auto >= vmin - eps) & (o_auto <= vmax + eps)).all())
    # oracle on the first KV head of the first batch row
    kk, vv = k[:1].cpu().reshape(1, 1, T, D), v[:1].cpu().reshape(1, 1, T, D)
    ref = ko.kivi_decode_attention(q[:1].cpu().reshape(1, n_rep, D), kk, vv, n_quant, G, "half_away", dtype=torch.float64)
    r0 = ref.float().reshape(1, n_rep, D)
    print(f"[cfg2 full size] unit 0 vs oracle: rel err {rel_err(o_auto[:1], r0):.2e}, element-wise {elem_err(o_auto[:1], r0):.2e}")
    assert rel_err(o_auto[:1], r0) < TOL_BF16


def test_full_size_config3_long_context(cabi):
    """The long-context shape: 32 units x (131072 quantized + 128 ring) tokens,
    bf16, split count chosen by the library (few units, so every unit is cut into
    many pieces).  One unit against the CPU oracle in fp64, agreement of the
    tensor-core and the fp32 kernel on two units, no bounded wait expired."""
    B, Hkv, n_rep, D, G, R, n_quant, n_res = 4, 8, 4, 128, 32, 128, 131072, 128
    U, T = B * Hkv, n_quant + n_res
    g = torch.Generator(device="cuda").manual_seed(321)
    k = torch.randn(U, T, D, device="cuda", generator=g)
    k[:, :, 17] *= 10.0
    k[:, :, 99] *= 10.0
    k = k.to(torch.bfloat16)
    v = torch.randn(U, T, D, device="cuda", generator=g)
    v *= 1.0 + 7.0 * (torch.rand(U, T, 1, device="cuda", generator=g) < 0.02)
    v = v.to(torch.bfloat16)
    st = cabi.LayerStore(U, D, G, R, n_quant, torch.bfloat16, "cuda")
    cabi.load_state(st, k, v, n_quant)
    q = torch.randn(U, n_rep, D, device="cuda", generator=g).to(torch.bfloat16)
    o_auto = st.attention(q, n_rep=n_rep, path=cabi.ATTN_MMA, out_dtype=torch.float32)
    o_s28 = st.attention(q, n_rep=n_rep, path=cabi.ATTN_MMA, num_splits=28, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert cabi.device_fault() == 0 and torch.isfinite(o_auto).all()
    assert rel_err(o_s28, o_auto) < TOL_BF16
    sub = slice(U - 2, U)
    st2 = cabi.LayerStore(2, D, G, R, n_quant, torch.bfloat16, "cuda")
    cabi.load_state(st2, k[sub], v[sub], n_quant)
    o_f32 = st2.attention(q[sub].contiguous(), n_rep=n_rep, path=cabi.ATTN_FP32, out_dtype=torch.float32)
    print(f"[cfg3 full size] tensor-core vs fp32 kernel {rel_err(o_auto[sub], o_f32):.2e}")
    assert rel_err(o_auto[sub], o_f32) < TOL_BF16
    u = 5
    kk, vv = k[u:u + 1].cpu().reshape(1, 1, T, D), v[u:u + 1].cpu().reshape(1, 1, T, D)
    ref = ko.kivi_decode_attention(q[u:u + 1].cpu().reshape(1, n_rep, D), kk, vv, n_quant, G, "half_away",
                                   dtype=torch.float64).float().reshape(1, n_rep, D)
    e_row, e_el = rel_err(o_auto[u:u + 1], ref), elem_err(o_auto[u:u + 1], ref)
    print(f"[cfg3 full size] unit {u} vs oracle: rel err {e_row:.2e}, element-wise {e_el:.2e}")
    assert e_row < TOL_BF16


def test_full_size_config4_prefill_properties(cabi):
    """Bulk prefill at the benchmark's full size (256 units, 8192 tokens, bf16):
    the round trip through the packed store stays within half a quantization
    step of the input for every element (step = the stored scale of its group),
    ring tokens come back exactly, and two sampled units equal the CPU oracle bit
    for bit (codes through the dequantized values, scales and zeros directly)."""
    U, S, D, G, R = 256, 8192, 128, 32, 128
    g = torch.Generator(device="cuda").manual_seed(77)
    k = torch.empty(U, S, D, device="cuda", dtype=torch.bfloat16)
    v = torch.empty(U, S, D, device="cuda", dtype=torch.bfloat16)
    for u0 in range(0, U, 64):
        k[u0:u0 + 64] = torch.randn(64, S, D, device="cuda", generator=g).to(torch.bfloat16)
        v[u0:u0 + 64] = torch.randn(64, S, D, device="cuda", generator=g).to(torch.bfloat16)
    k[:, :, 9] *= 10.0
    st = cabi.LayerStore(U, D, G, R, S, torch.bfloat16, "cuda")
    st.update(k, v)
    n_flush, ql, rl = cabi.cache_plan(0, 0, S, G, R)
    assert (st.quant_len, st.res_len) == (ql, rl) == (S - 96, 96)
    ng = ql // G
    for name, x, by_token in (("k", k, False), ("v", v, True)):
        served = st.materialize()[1 if by_token else 0]                     # fp32 [U, S, D]
        assert torch.equal(served[:, ql:], x[:, ql:].float()), f"{name}: ring tokens must come back exactly"
        if by_token:        # scale of (token t, channel group gd); stored rows are permuted inside 32-token blocks
            rows = st.v_scales[:, :ql].reshape(U, ng, 2, 4, 4, D // G).permute(0, 1, 2, 4, 3, 5).reshape(U, ql, D // G)
            step = rows.repeat_interleave(G, dim=2)
        else:               # scale of (group g, channel d)
            step = st.k_scales[:, :ng].repeat_interleave(G, dim=1)
        worst = 0.0
        for u0 in range(0, U, 32):                                           # bounded temporaries
            err = (served[u0:u0 + 32, :ql] - x[u0:u0 + 32, :ql].float()).abs()
            bound = step[u0:u0 + 32] * 0.5 * (1 + 1e-5) + 1e-30
            assert bool((err <= bound).all()), f"{name}: round trip off by more than half a step"
            worst = max(worst, float((err / step[u0:u0 + 32]).max()))
        print(f"[cfg4 full size] {name}: worst |error| / step = {worst:.4f}")
        del served, step
    # two units against the oracle
    for u in (3, 200):
        oc = ko.OracleCache(D, G, R, rounding="half_away")
        ku, vu = k[u].float().cpu().reshape(1, 1, S, D), v[u].float().cpu().reshape(1, 1, S, D)
        oc.append(ku, vu)
        sk, sv = oc.served()
        one = cabi.LayerStore(1, D, G, R, S, torch.bfloat16, "cuda")
        one.update(k[u:u + 1], v[u:u + 1])
        gk, gv = one.materialize()
        assert torch.equal(gk.cpu(), sk.reshape(1, S, D)) and torch.equal(gv.cpu(), sv.reshape(1, S, D))
        assert torch.equal(one.k_scales[0, :ng].cpu(), torch.stack(oc.k_scales, dim=2).reshape(ng, D))
        assert torch.equal(st.k_scales[u, :ng].cpu(), one.k_scales[0, :ng].cpu())
        assert torch.equal(st.v_codes[u, :ql].cpu(), one.v_codes[0, :ql].cpu())


@pytest.mark.parametrize("dtype,path", [(torch.bfloat16, "mma"), (torch.float32, "fp32")])
def test_attention_lse_combines_token_shards(cabi, dtype, path):
    """kivi_decode_attention_lse: the log-sum-exp equals the oracle's, and two
    stores holding disjoint token ranges of the same sequences (sequence
    sharding on one GPU) combine into the single-store result."""
    from intel_kivi_hybrid_b200.parallel import merge_token_shards
    B, H, n_rep, D, G, R = 1, 4, 4, 128, 32, 128
    n_quant, n_res, n1 = 1024, 77, 384
    T, U = n_quant + n_res, B * H
    K = ko.make_keys(B, H, T, D, seed=13)
    V = ko.make_values(B, H, T, D, seed=13)
    q = ko.make_queries(B, H * n_rep, D, seed=13)
    if dtype == torch.bfloat16:
        K, V, q = K.bfloat16().float(), V.bfloat16().float(), q.bfloat16().float()
    kc, vc = units(K).cuda().to(dtype), units(V).cuda().to(dtype)
    qd = q.reshape(U, n_rep, D).cuda().to(dtype)
    p = cabi.ATTN_MMA if path == "mma" else cabi.ATTN_FP32
    whole = cabi.LayerStore(U, D, G, R, n_quant, dtype, "cuda")
    cabi.load_state(whole, kc, vc, n_quant)
    out_w, lse_w = whole.attention_lse(qd, n_rep=n_rep, path=p, out_dtype=torch.float32)
    assert torch.equal(out_w, whole.attention(qd, n_rep=n_rep, path=p, out_dtype=torch.float32))
    # oracle log-sum-exp over the served cache
    kd, vd = whole.materialize()
    s = torch.einsum("uhd,utd->uht", qd.double().cpu(), kd.double().cpu()) * D ** -0.5
    assert torch.allclose(lse_w.cpu().double(), torch.logsumexp(s, -1), atol=2e-3 if dtype == torch.bfloat16 else 2e-5)
    # many pieces per unit: the fold done by a whole CTA per row gives the same log-sum-exp
    out_m, lse_m = whole.attention_lse(qd, n_rep=n_rep, path=p, out_dtype=torch.float32, num_splits=24)
    assert torch.allclose(lse_m, lse_w, atol=1e-5 if dtype == torch.float32 else 1e-4)
    assert rel_err(out_m, out_w) < (TOL_F32 if dtype == torch.float32 else TOL_BF16)
    # shard 0: the first n1 tokens, all quantized; shard 1: the rest with the ring
    s0 = cabi.LayerStore(U, D, G, R, n1, dtype, "cuda")
    cabi.load_state(s0, kc[:, :n1], vc[:, :n1], n1)
    s1 = cabi.LayerStore(U, D, G, R, n_quant - n1, dtype, "cuda")
    cabi.load_state(s1, kc[:, n1:], vc[:, n1:], n_quant - n1)
    o0, l0 = s0.attention_lse(qd, n_rep=n_rep, path=p, out_dtype=torch.float32)
    o1, l1 = s1.attention_lse(qd, n_rep=n_rep, path=p, out_dtype=torch.float32)
    merged = merge_token_shards(torch.stack([o0, o1]), torch.stack([l0, l1]))
    tol = TOL_BF16 if dtype == torch.bfloat16 else TOL_F32
    assert rel_err(merged, out_w) < tol
    ref = ko.kivi_decode_attention(q, K, V, n_quant, G, "half_away", dtype=torch.float64).float().reshape(U, n_rep, D)
    assert rel_err(merged, ref) < tol
    with pytest.raises(RuntimeError, match="empty cache"):
        cabi.LayerStore(U, D, G, R, 64, dtype, "cuda").attention_lse(qd, n_rep=n_rep)


@pytest.mark.parametrize("chunks,direct", [(1, True), (1, False), (2, False), (3, False)])
def test_decode_step_from_host_equals_update_then_attention(cabi, chunks, direct):
    """kivi_decode_step_host: pinned host q / new token in, pinned host output back.
    Over 40 steps (one flush inside) the counters, the packed store and the ring
    must end up bit-identical to update() + attention() called separately; the
    outputs are bit-identical with one chunk (same split plan) and within the
    tolerance of the oracle with several."""
    B, Hkv, n_rep, D, G, R = 2, 4, 4, 128, 32, 128
    U, T0, steps = B * Hkv, 700, 40
    K = ko.make_keys(B, Hkv, T0 + steps, D, seed=31).to(torch.bfloat16)
    V = ko.make_values(B, Hkv, T0 + steps, D, seed=31).to(torch.bfloat16)
    Kc, Vc = units(K).cuda(), units(V).cuda()
    a = cabi.LayerStore(U, D, G, R, 1024, torch.bfloat16, "cuda")
    b = cabi.LayerStore(U, D, G, R, 1024, torch.bfloat16, "cuda")
    a.update(Kc[:, :T0], Vc[:, :T0]); b.update(Kc[:, :T0], Vc[:, :T0])
    h_q = torch.empty(U, n_rep, D, dtype=torch.bfloat16).pin_memory()
    h_k = torch.empty(U, D, dtype=torch.bfloat16).pin_memory()
    h_v = torch.empty(U, D, dtype=torch.bfloat16).pin_memory()
    h_out = torch.empty(U, n_rep, D, dtype=torch.float32).pin_memory()
    worst = 0.0
    for t in range(T0, T0 + steps):
        q = ko.make_queries(B, Hkv * n_rep, D, seed=t).to(torch.bfloat16)
        h_q.copy_(q.reshape(U, n_rep, D)); h_k.copy_(units(K)[:, t]); h_v.copy_(units(V)[:, t])
        a.decode_step_host(h_q, h_k, h_v, h_out, n_rep, chunks=chunks, direct=direct)
        b.update(Kc[:, t:t + 1], Vc[:, t:t + 1])
        ref_out = b.attention(q.reshape(U, n_rep, D).cuda(), n_rep=n_rep, out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert (a.quant_len, a.res_start, a.res_len) == (b.quant_len, b.res_start, b.res_len)
        if chunks == 1:
            assert torch.equal(h_out, ref_out.cpu())
        else:
            assert rel_err(h_out, ref_out) < TOL_BF16
        if t % 13 == 0:
            ref = ko.kivi_decode_attention(q, K[:, :, :t + 1], V[:, :, :t + 1], a.quant_len, G, "half_away", dtype=torch.float64)
            worst = max(worst, rel_err(h_out, ref.float().reshape(U, n_rep, D)))
    assert a.quant_len == 640 and worst < TOL_BF16
    for name in ("k_codes", "k_scales", "k_zeros", "v_codes", "v_scales", "v_zeros", "k_res", "v_res"):
        assert torch.equal(getattr(a, name), getattr(b, name)), name
    assert cabi.device_fault() == 0
    with pytest.raises(RuntimeError, match="pinned"):
        a.decode_step_host(h_q.clone(), h_k, h_v, h_out, n_rep)


def test_tensor_core_keeps_enough_bits_for_subnormal_codes(cabi):
    """The tensor-core kernel feeds codes as fp16 subnormals; the MMA aligns its
    addends on their exponent fields and truncates a fixed distance below the
    largest.  The kernel's placement of the codes (no code lower than bits 2-3 of
    its half) leaves 20 bits if the unit keeps 26 below the largest addend's
    leading bit, i.e. still resolves 2^-25 next to 1."""
    bits = cabi.mma_alignment_bits()
    print(f"[tensor core] 1 + 2^-k - 1 is exact up to k = {bits}")
    assert bits >= 24
