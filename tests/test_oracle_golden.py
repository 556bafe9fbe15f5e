"""Pins the CPU oracle to vectors produced by the reference's own code
(tests/golden/make_golden.py) and to the known answers its tests hold."""
import os

import numpy as np
import pytest
import torch

from oracle import clib
from oracle import kivi_oracle as ko

CASES = ["rt_keys_seed0", "rt_values_seed1", "const5", "known_1234", "known_1234_x4",
         "g4", "g16", "g64", "g128", "g12", "bf16_derived", "cfg0_keys_flush", "cfg0_values"]


@pytest.fixture(scope="module")
def rt(golden_dir):
    return np.load(os.path.join(golden_dir, "roundtrip_vectors.npz"))


@pytest.mark.parametrize("name", CASES)
def test_restatement_equals_reference_mirror_bitwise(rt, name):
    x = torch.from_numpy(rt[name + "__x"])
    G = int(rt[name + "__G"])
    got = ko.roundtrip_groups(x, G, "half_even")
    assert torch.equal(got, torch.from_numpy(rt[name + "__mirror_rt"]))
    # quantize + dequantize == fused round trip (test_roundtrip_kernels.py:47,72)
    r = ko.quantize_groups(x, G, "half_even")
    deq = ko.dequantize_groups(r["packed"], r["scales"], r["zeros"], G).reshape(x.shape)
    assert torch.equal(deq, got)
    assert int(r["codes"].max()) <= 3


@pytest.mark.parametrize("name", CASES)
def test_half_away_restatements_equal_reference_kernel_header(rt, name):
    """torch half_away path and the plain-C port against the reference's own
    quant_tile.hpp (compiled through the shim when the golden file was made)."""
    x = torch.from_numpy(rt[name + "__x"])
    G = int(rt[name + "__G"])
    r = ko.quantize_groups(x, G, "half_away")
    assert np.array_equal(r["packed"].numpy(), rt[name + "__kernel_packed"])
    assert np.array_equal(r["scales"].numpy(), rt[name + "__kernel_scales"])
    assert np.array_equal(r["zeros"].numpy(), rt[name + "__kernel_zeros"])
    assert np.array_equal(ko.roundtrip_groups(x, G, "half_away").numpy(), rt[name + "__kernel_rt"])
    pk, sc, zr = clib.c_quantize(x.numpy(), G, half_even=False)
    assert np.array_equal(pk, rt[name + "__kernel_packed"])
    assert np.array_equal(sc, rt[name + "__kernel_scales"])
    assert np.array_equal(zr, rt[name + "__kernel_zeros"])
    assert np.array_equal(clib.c_roundtrip(x.numpy(), G, False), rt[name + "__kernel_rt"])
    assert np.array_equal(clib.c_dequantize(pk, sc, zr, G).reshape(x.shape), rt[name + "__kernel_rt"])
    # C port in half-even mode == torch mirror
    assert np.array_equal(clib.c_roundtrip(x.numpy(), G, True), rt[name + "__mirror_rt"])


@pytest.mark.parametrize("name", CASES)
def test_conventions_differ_only_at_exact_ties(rt, name):
    x = torch.from_numpy(rt[name + "__x"])
    G = int(rt[name + "__G"])
    even = ko.quantize_groups(x, G, "half_even")["codes"]
    away = ko.quantize_groups(x, G, "half_away")["codes"]
    ties = ko.tie_mask(x.reshape(-1, G)).reshape(-1)
    assert torch.equal(even[~ties], away[~ties])
    if name == "bf16_derived":
        assert int(ties.sum()) > 0      # ~1e-3 per element on bf16-derived data


def test_known_answers(rt):
    # [1,2,3,4], G=4 -> scale 1.0, zero 1.0, byte 228 (test_kivi.py:160-196)
    r = ko.quantize_groups(torch.tensor([1.0, 2.0, 3.0, 4.0]), 4)
    assert r["packed"].tolist() == [228] and r["scales"].item() == 1.0 and r["zeros"].item() == 1.0
    assert ko.dequantize_groups(r["packed"], r["scales"], r["zeros"], 4).tolist() == [1.0, 2.0, 3.0, 4.0]
    assert rt["known_1234__kernel_packed"].tolist() == [228]
    # constant input: scale 1e-10, codes 0, dequant exactly 5.0 (test_roundtrip_kernels.py:79-87)
    c = ko.quantize_groups(torch.full((128,), 5.0), 32)
    assert torch.all(c["codes"] == 0) and torch.all(c["scales"] == np.float32(1e-10))
    assert torch.all(ko.roundtrip_groups(torch.full((128,), 5.0), 32) == 5.0)
    # error bound the reference tests use: <= 0.6 * max scale (test_kivi.py:82)
    x = torch.from_numpy(rt["rt_keys_seed0__x"])
    q = ko.quantize_groups(x, 32)
    err = (ko.roundtrip_groups(x, 32) - x).abs().max()
    assert err <= 0.6 * q["scales"].max()


def test_state_machine_matches_reference_cache(golden_dir):
    sm = np.load(os.path.join(golden_dir, "state_machine_vectors.npz"))
    steps, prefill, G, R, D, layers, heads = [int(v) for v in sm["params"]]
    for mode in ("in_place", "legacy_tuple"):
        for i in range(layers):
            truth_k = torch.from_numpy(sm[f"{mode}__truth_k{i}"])
            oc = ko.OracleCache(D, G, R)
            oc.append(truth_k[:, :, :prefill], truth_k[:, :, :prefill])
            for t in range(prefill, prefill + steps):
                oc.append(truth_k[:, :, t:t + 1], truth_k[:, :, t:t + 1])
            sk, _ = oc.served()
            assert torch.equal(sk, torch.from_numpy(sm[f"{mode}__served_k{i}"]))
            assert oc.quantized_len == int(sm[f"{mode}__quant_tokens"][i])
        assert int(sm[f"{mode}__total_flushes"]) == layers * (int(sm[f"{mode}__quant_tokens"][0]) // G)
    # longer run: 200-token prefill then 100 single-token appends, G=32, R=128
    K, V = torch.from_numpy(sm["long__K"]), torch.from_numpy(sm["long__V"])
    oc = ko.OracleCache(64, 32, 128)
    oc.append(K[:, :, :200], V[:, :, :200])
    for t in range(200, 300):
        oc.append(K[:, :, t:t + 1], V[:, :, t:t + 1])
    sk, sv = oc.served()
    assert torch.equal(sk, torch.from_numpy(sm["long__served_k"]))
    assert torch.equal(sv, torch.from_numpy(sm["long__served_v"]))
    assert oc.quantized_len == int(sm["long__quant_tokens"])
    assert oc.flushes == int(sm["long__total_flushes"])
    f, ql, rl = ko.flush_schedule(0, 0, 200, 32, 128)
    assert (f, ql, rl) == (3, 96, 104)
    # analytic byte accounting (manager.py:350-356) and compression figure
    res_bytes = 2 * oc.res_k.numel() * 4
    assert oc.stats_bytes() + res_bytes == int(sm["long__stat_kivi_bytes"])
    # prefill of S >= R triggers floor((S-R)/G)+1 flushes; S=512 -> 13, 416 + 96
    assert ko.flush_schedule(0, 0, 512, 32, 128) == (13, 416, 96)


def test_attention_matches_reference_formula(golden_dir):
    av = np.load(os.path.join(golden_dir, "attention_vectors.npz"))
    q, k, v = (torch.from_numpy(av[n]) for n in ("query", "key", "value"))
    assert torch.allclose(ko.attention(q, k, v), torch.from_numpy(av["out_fp32"]), atol=1e-6)
    # every query position separately through the decode composition
    for i in range(q.shape[2]):
        out = ko.kivi_decode_attention(q[:, :, i], k, v, n_quant=32, group_size=32)
        ref = torch.from_numpy(av["out_kivi"])[:, :, i]
        assert torch.allclose(out, ref, atol=2e-6, rtol=1e-5)
    assert av["cosine"] > 0.85          # the reference's own pass threshold
    # grouped-query evaluation == explicit repetition of KV heads
    g = torch.Generator().manual_seed(3)
    qq = torch.randn(2, 8, 1, 16, generator=g)
    kk = torch.randn(2, 2, 40, 16, generator=g)
    vv = torch.randn(2, 2, 40, 16, generator=g)
    rep = ko.attention(qq, kk.repeat_interleave(4, dim=1), vv.repeat_interleave(4, dim=1))
    assert torch.allclose(ko.attention(qq, kk, vv), rep, atol=1e-6)
