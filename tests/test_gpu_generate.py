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


def test_fused_attention_hook_matches_oracle_after_flushes():
    """With a 32-token window the hook flushes every 32 tokens.  Every decode
    step's attention output (each layer) is compared with the CPU oracle fed the
    very K/V tensors the model produced: the tokens before the step's
    quantized length round-tripped group by group, the rest exact."""
    from kivi_sycl import KiviCache
    from intel_kivi_hybrid_b200.generation.hf_attention import attached
    from oracle import kivi_oracle as ko
    model = _model("cuda")
    G = R = 32
    cache = KiviCache.from_model(model, device="cuda", group_size=G, residual_length=R)
    seen_k = [[] for _ in range(cache.num_layers)]
    seen_v = [[] for _ in range(cache.num_layers)]
    calls = []
    ingest, attend = cache.ingest_layer, cache.decode_attention

    def rec_ingest(layer, k, v):
        seen_k[layer].append(k.detach().float().cpu()); seen_v[layer].append(v.detach().float().cpu())
        return ingest(layer, k, v)

    def rec_attend(layer, q, **kw):
        out = attend(layer, q, **kw)
        calls.append((layer, q.detach().float().cpu(), out.detach().float().cpu(), cache._quant_token_count[layer]))
        return out

    cache.ingest_layer, cache.decode_attention = rec_ingest, rec_attend
    ids = torch.tensor([[3 + i % 90 for i in range(40)]], device="cuda")
    with torch.no_grad(), attached(model, cache) as pkv:
        model(ids, past_key_values=pkv, use_cache=True)
        for i in range(60):
            model(torch.tensor([[5 + i % 80]], device="cuda"), past_key_values=pkv, use_cache=True)
    assert len(calls) == 60 * cache.num_layers and cache.total_flushes == 3 * cache.num_layers
    worst, flushed_steps = 0.0, 0
    for n, (layer, q, out, n_quant) in enumerate(calls):
        T = 40 + n // cache.num_layers + 1                      # tokens the cache held when this step attended
        K = torch.cat(seen_k[layer], dim=2)[:, :, :T]
        V = torch.cat(seen_v[layer], dim=2)[:, :, :T]
        assert n_quant % G == 0 and 0 <= T - n_quant < R
        ref = ko.kivi_decode_attention(q, K, V, n_quant, G, "half_away", dtype=torch.float64).float()
        err = float(((out - ref).abs().amax(-1) / ref.abs().amax(-1)).max())
        worst = max(worst, err)
        flushed_steps += n_quant > 32
    print(f"[fused hook, {flushed_steps} steps after the second flush] worst rel err vs oracle {worst:.2e}")
    assert flushed_steps > 0 and worst < 1e-5


def test_fused_attention_hook_refuses_chunked_prefill():
    """Several query tokens on a cache that already holds tokens would ignore the
    packed history: the hook must raise, not attend over the new tokens alone."""
    from kivi_sycl import KiviCache
    from intel_kivi_hybrid_b200.generation.hf_attention import attached
    model = _model("cuda")
    ids = torch.tensor([[3 + i % 90 for i in range(24)]], device="cuda")
    cache = KiviCache.from_model(model, device="cuda", group_size=32, residual_length=128)
    with torch.no_grad(), attached(model, cache) as pkv:
        model(ids[:, :12], past_key_values=pkv, use_cache=True)
        with pytest.raises(RuntimeError, match="chunked prefill"):
            model(ids[:, 12:], past_key_values=pkv, use_cache=True)


def test_generate_stops_at_eos_like_the_reference_loop():
    """EOS is looked for every few steps on the device-resident ids; the text
    must still end with the first EOS, as the reference's per-step test gives."""
    from kivi_sycl import generate
    model, tok = _model("cuda"), _Tok()
    prompt = " ".join(str(i % 97) for i in range(3, 23))
    ids = tok(prompt).input_ids.cuda()
    with torch.no_grad():
        plain = model.generate(ids, max_new_tokens=40, do_sample=False, pad_token_id=0)[0].tolist()
    new = plain[20:]
    for pos in (0, 5, 11, 17):                      # an EOS at the first token, inside and at the edge of a check window
        eos = _Tok()
        eos.eos_token_id = new[pos]
        first = new.index(new[pos])
        want = " ".join(str(t) for t in plain[:20 + first + 1])
        for fused in (False, True):
            got = generate(model, eos, prompt, max_new_tokens=40, residual_length=128, device="cuda", fused_attention=fused)
            assert got == want, (pos, fused)
