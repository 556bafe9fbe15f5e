"""generate() end to end with a randomly initialised GPT-2 (no weights needed):
while nothing has been flushed the KIVI pipeline must reproduce plain greedy
decoding token for token (the check examples/cpu_sim.py --identity makes in the
reference); with a small window it must keep running through many flushes."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


class _Tok:
    eos_token_id = None

    def __call__(self, prompt, return_tensors="pt"):
        ids = torch.tensor([[int(t) for t in prompt.split()]])
        return types.SimpleNamespace(input_ids=ids)

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(t)) for t in ids)


def _model(device):
    from transformers import GPT2Config, GPT2LMHeadModel
    torch.manual_seed(0)
    cfg = GPT2Config(n_layer=2, n_head=2, n_embd=64, vocab_size=97, n_positions=256)
    return GPT2LMHeadModel(cfg).eval().to(device)


@pytest.mark.parametrize("model_device", ["cuda", "cpu"])
def test_generate_matches_plain_greedy_before_any_flush(model_device):
    from kivi_sycl import generate
    model, tok = _model(model_device), _Tok()
    prompt = " ".join(str(i % 97) for i in range(3, 23))
    ids = tok(prompt).input_ids.to(model_device)
    with torch.no_grad():
        ref = model.generate(ids, max_new_tokens=30, do_sample=False, pad_token_id=0)[0]
    text = generate(model, tok, prompt, max_new_tokens=30, group_size=32, residual_length=128, device="cuda")
    assert text == tok.decode(ref)


def test_generate_runs_through_flushes_and_sampling():
    from kivi_sycl import KiviCache, generate
    model, tok = _model("cuda"), _Tok()
    prompt = " ".join(str(i % 97) for i in range(40))
    text = generate(model, tok, prompt, max_new_tokens=60, group_size=32, residual_length=32, device="cuda")
    assert len(text.split()) == 100
    torch.manual_seed(1)
    text = generate(model, tok, prompt, max_new_tokens=20, group_size=32, residual_length=64, device="cuda",
                    temperature=0.8, top_k=5, do_sample=True)
    assert len(text.split()) == 60
    cache = KiviCache.from_model(model, device="cuda", group_size=32, residual_length=32)
    assert (cache.num_layers, cache.head_dim, cache.num_kv_heads) == (2, 32, 2)


def test_fused_attention_hook_reproduces_model_logits():
    """generate(fused_attention=True): the model's K/V stream into the cache and
    decode steps attend through the fused kernel.  Before any flush the logits
    must equal the plain model's to fp32 rounding."""
    from kivi_sycl import KiviCache
    from intel_kivi_hybrid_b200.generation.hf_attention import attached
    model = _model("cuda")
    ids = torch.tensor([[3 + i % 90 for i in range(24)]], device="cuda")
    steps = [torch.tensor([[11 + i]], device="cuda") for i in range(4)]
    with torch.no_grad():
        ref = model(ids, use_cache=True)
        ref_logits = [ref.logits[:, -1]]
        past = ref.past_key_values
        for t in steps:
            o = model(t, past_key_values=past, use_cache=True)
            ref_logits.append(o.logits[:, -1]); past = o.past_key_values
        cache = KiviCache.from_model(model, device="cuda", group_size=32, residual_length=128)
        got = []
        with attached(model, cache) as pkv:
            o = model(ids, past_key_values=pkv, use_cache=True); got.append(o.logits[:, -1])
            for t in steps:
                o = model(t, past_key_values=pkv, use_cache=True); got.append(o.logits[:, -1])
        assert model.config._attn_implementation != "kivi_fused"          # restored
    assert cache._stores[0].res_len == 28 and cache._quant_token_count == [0, 0]
    for a, b in zip(got, ref_logits):
        assert torch.allclose(a, b, atol=2e-4, rtol=1e-4), (a - b).abs().max()


def test_generate_with_fused_attention_runs_through_flushes():
    from kivi_sycl import generate
    model, tok = _model("cuda"), _Tok()
    prompt = " ".join(str(i % 97) for i in range(40))
    text = generate(model, tok, prompt, max_new_tokens=60, group_size=32, residual_length=32, device="cuda",
                    fused_attention=True)
    assert len(text.split()) == 100
    # same tokens as the dense-cache path while nothing has been flushed
    short = " ".join(str(i % 97) for i in range(3, 23))
    a = generate(model, tok, short, max_new_tokens=20, residual_length=128, device="cuda", fused_attention=True)
    b = generate(model, tok, short, max_new_tokens=20, residual_length=128, device="cuda")
    assert a == b
