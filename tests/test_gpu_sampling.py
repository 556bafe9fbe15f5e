"""Device-side next-token choice (kivi_sample_tokens) against torch and the CPU
restatement: argmax bit-exact (ties to the lowest index), top_k = 1 equal to the
argmax, the counter-based draws reproduced by the oracle, the distribution of
1e5 draws against the exact softmax (chi-square), repeatability."""
import pytest
import torch

from oracle import kivi_oracle as ko

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cabi():
    from intel_kivi_hybrid_b200 import cabi as m
    return m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_argmax_equals_torch(cabi, dtype):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(9, 50257, generator=g).to(dtype)
    x[2, 40000] = x[2, 17] = x[2].max() + 1           # a tie: the lower index wins
    x[5, :] = 0.25                                    # a constant row
    ids = cabi.sample_tokens(x.cuda(), do_sample=False)
    assert torch.equal(ids.cpu(), x.float().argmax(dim=-1)) and int(ids[2]) == 17 and int(ids[5]) == 0
    # a view with a row stride (the last position of [B, L, V] logits)
    full = torch.randn(4, 3, 1000, generator=g).to(dtype).cuda()
    assert torch.equal(cabi.sample_tokens(full[:, -1, :], do_sample=False), full[:, -1, :].float().argmax(dim=-1))


def test_top_k_one_is_the_argmax_and_draws_repeat(cabi):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(32, 32000, generator=g).cuda()
    a = cabi.sample_tokens(x, temperature=0.7, top_k=1, do_sample=True, seed=11, step=3)
    assert torch.equal(a, x.argmax(dim=-1))
    b = cabi.sample_tokens(x, temperature=1.3, top_k=40, do_sample=True, seed=11, step=3)
    c = cabi.sample_tokens(x, temperature=1.3, top_k=40, do_sample=True, seed=11, step=3)
    d = cabi.sample_tokens(x, temperature=1.3, top_k=40, do_sample=True, seed=11, step=4)
    assert torch.equal(b, c) and not torch.equal(b, d)
    kept = x.topk(40, dim=-1).indices
    assert bool((kept == b[:, None]).any(dim=1).all())          # every draw lies inside the top 40


@pytest.mark.parametrize("top_k,temperature", [(None, 1.0), (50, 0.8), (5, 2.5)])
def test_draws_are_reproduced_by_the_oracle(cabi, top_k, temperature):
    g = torch.Generator().manual_seed(5)
    x = (3.0 * torch.randn(64, 5000, generator=g))
    got = cabi.sample_tokens(x.cuda(), temperature, top_k or 0, True, seed=2**40 + 7, step=9).cpu()
    want = ko.sample_tokens(x, temperature, top_k, True, seed=2**40 + 7, step=9)
    # identical uniform numbers; the masses are summed in fp32-exp / fp64-sum on both
    # sides but exp differs in the last bit, so a draw that lands on a boundary may
    # move to the neighbour: at most one row may differ
    assert int((got != want).sum()) <= 1, (got, want)


def test_distribution_of_draws_matches_softmax(cabi):
    V, N = 40, 100000
    g = torch.Generator().manual_seed(6)
    row = 1.5 * torch.randn(V, generator=g)
    x = row.repeat(N, 1).cuda()
    ids = cabi.sample_tokens(x, temperature=0.9, top_k=0, do_sample=True, seed=123, step=0).cpu()
    p = torch.softmax(row.double() / 0.9, dim=-1)
    counts = torch.bincount(ids, minlength=V).double()
    chi2 = float(((counts - N * p) ** 2 / (N * p)).sum())
    print(f"[sampling] chi-square over {N} draws, {V - 1} degrees of freedom: {chi2:.1f}")
    assert chi2 < 85.0                                           # p ~ 3e-5 for 39 degrees of freedom
    torch.manual_seed(0)
    ref = torch.multinomial(p.float().cuda().repeat(N, 1), 1)[:, 0].cpu()
    chi2_t = float(((torch.bincount(ref, minlength=V).double() - N * p) ** 2 / (N * p)).sum())
    print(f"[sampling] torch.multinomial on the same probabilities: {chi2_t:.1f}")


def test_sample_token_keeps_ids_on_the_device_and_validates(cabi):
    from intel_kivi_hybrid_b200.generation.sampling import sample_token
    x = torch.randn(2, 97).cuda()
    ids = sample_token(x, 1.0, None, False)
    assert ids.is_cuda and ids.shape == (2, 1) and torch.equal(ids[:, 0], x.argmax(dim=-1))
    torch.manual_seed(5)
    a = [sample_token(x, 0.8, 10, True) for _ in range(3)]
    torch.manual_seed(5)
    b = [sample_token(x, 0.8, 10, True) for _ in range(3)]
    assert all(torch.equal(i, j) for i, j in zip(a, b))          # torch.manual_seed makes a run repeatable
    with pytest.raises(RuntimeError, match="CUDA device"):
        cabi.sample_tokens(torch.randn(2, 8))
    with pytest.raises(RuntimeError, match="top_k"):
        cabi.sample_tokens(x, top_k=-1, do_sample=True)
