"""kivi_decode_attention_noalloc: the variant of decode attention for hosts that
may not allocate device memory (a server whose pool owns all of HBM, a plug-in
inside another framework's memory plan).  Its split partials sit in a fixed
array inside the library instead of a caller workspace.

Collected last on purpose (file name): if it fails, a run that stops at the
first failure has already run every other test.  Checks, through the C ABI, that
two calls in a row give what the workspace-taking entry point gives, that the
shared array needs no clearing between different problems, and that a problem
beyond the array's size is refused with a message naming the limit."""
import pytest
import torch

from oracle import kivi_oracle as ko

pytestmark = pytest.mark.gpu


def _store(cabi, B, Hkv, D, n_quant, n_res, seed, dtype=torch.bfloat16):
    T = n_quant + n_res
    K = ko.make_keys(B, Hkv, T, D, seed).to(dtype)
    V = ko.make_values(B, Hkv, T, D, seed).to(dtype)
    st = cabi.LayerStore(B * Hkv, D, 32, 128, max(n_quant, 32), dtype, "cuda")
    cabi.load_state(st, K.reshape(B * Hkv, T, D).cuda(), V.reshape(B * Hkv, T, D).cuda(), n_quant)
    return st


def test_noalloc_entry_point_matches_workspace_entry_point():
    from intel_kivi_hybrid_b200 import cabi
    n_rep, D = 4, 128
    big = _store(cabi, 2, 8, D, 3968, 128, seed=41)
    small = _store(cabi, 1, 2, D, 96, 37, seed=42)
    for st, path in ((big, cabi.ATTN_MMA), (small, cabi.ATTN_FP32), (big, cabi.ATTN_FP32), (small, cabi.ATTN_MMA)):
        q = torch.randn(st.num_units, n_rep, D, device="cuda").to(torch.bfloat16)
        ref = st.attention(q, n_rep=n_rep, path=path, out_dtype=torch.float32)
        out1 = torch.full_like(ref, float("nan"))
        out2 = torch.full_like(ref, float("nan"))
        before = torch.cuda.memory_allocated()
        st.attention_noalloc(q, out1, n_rep, path=path)          # two calls in a row on the shared array
        st.attention_noalloc(q, out2, n_rep, path=path)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before           # nothing went through torch's allocator
        # same kernels, same split plan, same order of additions: identical bits
        assert torch.isfinite(out1).all() and torch.isfinite(out2).all()
        assert torch.equal(out1, ref) and torch.equal(out2, ref)
    assert cabi.device_fault() == 0


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from intel_kivi_hybrid_b200 import cabi
    D, n_rep = 128, 4
    st = cabi.LayerStore(1024, D, 32, 128, 128 * 32, torch.bfloat16, "cuda")
    st.quant_len, st.res_len = 128 * 32, 0                        # contents irrelevant: refused before any launch
    q = torch.zeros(1024, n_rep, D, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(1024, n_rep, D, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        st.attention_noalloc(q, out, n_rep, num_splits=64)       # 1024*64*4*130*4 B = 136 MB > 8 MiB
    st.attention_noalloc(q, out, n_rep, num_splits=2)            # 4.3 MB: accepted
    torch.cuda.synchronize()
