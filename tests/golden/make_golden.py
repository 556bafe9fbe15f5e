"""Generates tests/golden/*.npz by running the REFERENCE's own code.

Run once on a machine that has the reference tree:

    python tests/golden/make_golden.py /path/to/reference      (or set KIVI_REFERENCE_DIR)

What is imported from the reference (never copied):
  * examples/cpu_sim.py::_roundtrip_2bit                       (torch mirror)
  * tests/unit/test_manager_bookkeeping.py::_roundtrip_2bit_reference,
    FakeModel, and through it the real kivi_sycl.cache.manager.KiviCache with
    the reference's own stand-in for the native module
  * oracle/_ref/libkivi_ref_tile.so, i.e. the reference's quant_tile.hpp
    compiled by oracle/Makefile (device-kernel rounding: half away from zero)
The attention vector re-creates the inputs of
tests/integration/test_attention_fix.py (seed 42, B=1,H=2,q_len=3,cache_len=32,
D=64,G=32; that script needs an XPU at import, so it is read, not imported) and
applies the formula written there to the mirror-round-tripped K/V.
Inputs are stored too, so the tests need neither the reference nor this script.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
from oracle import clib  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else clib.reference_dir()
if not REF:
    sys.exit("usage: make_golden.py <reference tree>  (or set KIVI_REFERENCE_DIR)")


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    clib.build(REF)
    cpu_sim = _load(os.path.join(REF, "examples", "cpu_sim.py"), "ref_cpu_sim")
    sys.path.insert(0, os.path.join(REF, "src"))
    tmb = _load(os.path.join(REF, "tests", "unit", "test_manager_bookkeeping.py"), "ref_tmb")

    def mirror(x, G):
        out = torch.empty_like(x)
        cpu_sim._roundtrip_2bit(x, out, G)
        out2 = torch.empty_like(x)
        tmb._roundtrip_2bit_reference(x, out2, G)
        assert torch.equal(out, out2), "the reference's two mirrors disagree"
        return out

    # ---------------- round-trip / quantize vectors -----------------------
    cases = {}

    def add_case(name, x, G):
        x = x.contiguous()
        rt = mirror(x, G)
        pk, sc, zr = clib.ref_quantize(x.numpy(), G)
        rt_dev = clib.ref_roundtrip(x.numpy(), G)
        cases[name + "__x"] = x.numpy()
        cases[name + "__G"] = np.int32(G)
        cases[name + "__mirror_rt"] = rt.numpy()            # torch mirror (half even)
        cases[name + "__kernel_packed"] = pk                # quant_tile.hpp (half away)
        cases[name + "__kernel_scales"] = sc
        cases[name + "__kernel_zeros"] = zr
        cases[name + "__kernel_rt"] = rt_dev

    torch.manual_seed(0)      # tests/integration/test_roundtrip_kernels.py:30-33
    add_case("rt_keys_seed0", torch.randn(2, 3, 64, 32), 32)
    torch.manual_seed(1)      # tests/integration/test_roundtrip_kernels.py:55-58
    add_case("rt_values_seed1", torch.randn(2, 3, 8, 64), 32)
    add_case("const5", torch.full((1, 1, 4, 32), 5.0), 32)   # test_roundtrip_kernels.py:79-87
    add_case("known_1234", torch.tensor([[[[1.0, 2.0, 3.0, 4.0]]]]), 4)  # test_kivi.py:160-196
    add_case("known_1234_x4", torch.tensor([1.0, 2.0, 3.0, 4.0]).repeat(1, 1, 4, 1), 4)  # test_quantize_simple.py
    g = torch.Generator().manual_seed(7)
    add_case("g4", torch.randn(3, 5, 8, 4, generator=g), 4)
    add_case("g16", torch.randn(2, 2, 16, 64, generator=g), 16)
    add_case("g64", torch.randn(2, 2, 4, 128, generator=g), 64)
    add_case("g128", torch.randn(1, 2, 6, 128, generator=g), 128)
    add_case("g12", torch.randn(2, 24, generator=g), 12)
    # bf16-derived inputs: many exact round-half ties
    xb = torch.randn(4, 8, 64, 32, generator=g).to(torch.bfloat16).float()
    add_case("bf16_derived", xb, 32)
    # outlier channels (keys, [B,H,D,S] flush-shaped) and outlier tokens
    from oracle import kivi_oracle as ko
    k = ko.make_keys(1, 12, 32, 64, seed=100).transpose(2, 3).contiguous()
    add_case("cfg0_keys_flush", k, 32)
    v = ko.make_values(1, 12, 64, 64, seed=100)
    add_case("cfg0_values", v, 32)
    np.savez_compressed(os.path.join(HERE, "roundtrip_vectors.npz"), **cases)

    # ---------------- state machine vectors -------------------------------
    sm = {}
    for mode in ("in_place", "legacy_tuple"):
        torch.manual_seed(11)
        cache, model = tmb._run_generation(mode, identity=False)
        served = list(tmb._iter_kv_layers(cache.get_full_cache()))
        for i, (k_, v_) in enumerate(served):
            sm[f"{mode}__served_k{i}"] = k_.numpy()
            sm[f"{mode}__served_v{i}"] = v_.numpy()
            sm[f"{mode}__truth_k{i}"] = model.truth[i].numpy()
        # FakeModel keeps only key truth; values are base - jitter = 2*base - key
        sm[f"{mode}__quant_tokens"] = np.array(cache._quant_token_count)
        sm[f"{mode}__total_flushes"] = np.int64(cache.total_flushes)
        st = cache.get_stats(0)
        for key, val in st.items():
            sm[f"{mode}__stat_{key}"] = np.float64(val)
    sm["params"] = np.array([24, 6, 4, 8, 8, 2, 2])  # steps, prefill, G, R, D, layers, heads
    # a longer run at config-0-like flush parameters, driven token by token
    torch.manual_seed(12)
    tmb._fake_native.identity = False
    KiviCache = tmb.KiviCache
    cache = KiviCache(num_layers=1, head_dim=64, num_kv_heads=3, device="cpu",
                      group_size=32, residual_length=128)
    g2 = torch.Generator().manual_seed(13)
    K = torch.randn(1, 3, 300, 64, generator=g2)
    V = torch.randn(1, 3, 300, 64, generator=g2)
    cache.add_tokens(((K[:, :, :200], V[:, :, :200]),))
    for t in range(200, 300):
        cache.add_tokens(((K[:, :, :t + 1], V[:, :, :t + 1]),))
    sk, sv = next(iter(tmb._iter_kv_layers(cache.get_full_cache())))
    sm["long__K"] = K.numpy()
    sm["long__V"] = V.numpy()
    sm["long__served_k"] = sk.numpy()
    sm["long__served_v"] = sv.numpy()
    sm["long__quant_tokens"] = np.int64(cache._quant_token_count[0])
    sm["long__total_flushes"] = np.int64(cache.total_flushes)
    for key, val in cache.get_stats(0).items():
        sm[f"long__stat_{key}"] = np.float64(val)
    np.savez_compressed(os.path.join(HERE, "state_machine_vectors.npz"), **sm)

    # ---------------- attention vector -------------------------------------
    torch.manual_seed(42)       # test_attention_fix.py:33-36
    B, H, Lq, T, D, G = 1, 2, 3, 32, 64, 32
    query = torch.randn(B, H, Lq, D)
    key = torch.randn(B, H, T, D)
    value = torch.randn(B, H, T, D)
    sf = D ** -0.5              # test_attention_fix.py:40-43
    w = torch.softmax(torch.matmul(query, key.transpose(-2, -1)) * sf, dim=-1)
    out_fp32 = torch.matmul(w, value)
    k_deq = mirror(key.transpose(2, 3).contiguous(), G).transpose(2, 3)
    v_deq = mirror(value.contiguous(), G)
    w = torch.softmax(torch.matmul(query, k_deq.transpose(-2, -1)) * sf, dim=-1)   # :91-93
    out_kivi = torch.matmul(w, v_deq)
    cos = torch.nn.functional.cosine_similarity(out_fp32.reshape(1, -1), out_kivi.reshape(1, -1)).item()
    np.savez_compressed(os.path.join(HERE, "attention_vectors.npz"),
                        query=query.numpy(), key=key.numpy(), value=value.numpy(),
                        out_fp32=out_fp32.numpy(), out_kivi=out_kivi.numpy(),
                        cosine=np.float64(cos))
    print("cosine(seed 42) =", cos)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
