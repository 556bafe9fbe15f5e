"""Sharded KiviCache on two GPUs (skipped when fewer are visible): every rank
keeps half of the (batch, kv_head) units, the all-gathered decode-attention
output must equal the single-GPU output bit for bit (same kernel, same number
of splits per unit) and the oracle within tolerance; the same holds when the
all-gather happens inside the attention's last kernel through peer-mapped memory
(gather="peer", three calls in a row so that both halves of the double buffer
and the epoch flags are exercised).  Ranks are child processes over NCCL; each
leaves only after its last collective has completed.  A world of one (gloo, one
GPU) runs the same peer-gather kernel without peers."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r'''
import os, sys, datetime, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from kivi_cuda import KiviCache
from oracle import kivi_oracle as ko
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = f"cuda:{rank}"
if world > 1:
    dist.init_process_group("nccl", device_id=torch.device(dev), timeout=datetime.timedelta(seconds=60))
else:
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
B, Hkv, n_rep, D, T = 2, 4, 4, 128, 650
K = ko.make_keys(B, Hkv, T, D, 5).to(torch.bfloat16)
V = ko.make_values(B, Hkv, T, D, 5).to(torch.bfloat16)
q = ko.make_queries(B, Hkv * n_rep, D, 5).to(torch.bfloat16)
sharded = KiviCache(num_layers=1, head_dim=D, device=dev, shard=(rank, world))
single = KiviCache(num_layers=1, head_dim=D, device=dev)
for c in (sharded, single):
    c.add_tokens(((K[:, :, :T - 3].to(dev), V[:, :, :T - 3].to(dev)),))
    c.add_tokens(((K.to(dev), V.to(dev)),))
assert sharded._stores[0].num_units == B * Hkv // world
out_s = sharded.decode_attention(0, q.to(dev), out_dtype=torch.float32, num_splits=3)
out_1 = single.decode_attention(0, q.to(dev), out_dtype=torch.float32, num_splits=3)
torch.cuda.synchronize()
assert torch.equal(out_s, out_1), "sharded output differs from the single-GPU output"
ref = ko.kivi_decode_attention(q, K, V, single._quant_token_count[0], 32, "half_away", dtype=torch.float64).float()
err = ((out_s.cpu() - ref).abs().amax(-1) / ref.abs().amax(-1)).max().item()
assert err < 2e-3, err
from intel_kivi_hybrid_b200 import cabi
if world == 1:
    # a world of one: the gather kernel, the shared allocation and the flags, no peer
    from intel_kivi_hybrid_b200.parallel import PeerGather
    pg = PeerGather(B * Hkv, n_rep, D, torch.float32, 0, 1)
    st = single._stores[0]
    for _ in range(3):
        st.attention_gather(q.to(dev).reshape(B * Hkv, n_rep, D), pg.descriptor(), torch.float32, n_rep, num_splits=3)
        torch.cuda.synchronize()
        assert torch.equal(pg.gathered().reshape(B, Hkv * n_rep, D), out_1), "peer-gather output differs"
    # the host-to-host decode step through the same exchange: pinned q / new token in,
    # the gathered rows back in pinned memory (what bench.py's end-to-end loop calls at N > 1)
    twin = KiviCache(num_layers=1, head_dim=D, device=dev)
    twin.add_tokens(((K[:, :, :T - 3].to(dev), V[:, :, :T - 3].to(dev)),))
    twin.add_tokens(((K.to(dev), V.to(dev)),))
    a, b = st, twin._stores[0]
    U = B * Hkv
    h_q = q.reshape(U, n_rep, D).contiguous().pin_memory()
    h_k = torch.randn(U, D).to(torch.bfloat16).pin_memory()
    h_v = torch.randn(U, D).to(torch.bfloat16).pin_memory()
    h_out = torch.empty(U, n_rep, D, dtype=torch.float32).pin_memory()
    for direct in (True, False):
        a.decode_step_host(h_q, h_k, h_v, h_out, n_rep, num_splits=3, direct=direct, gather=pg.descriptor(), gather_units=U)
        b.update(h_k.to(dev).unsqueeze(1), h_v.to(dev).unsqueeze(1))
        want = b.attention(h_q.to(dev), n_rep=n_rep, num_splits=3, out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert (a.quant_len, a.res_start, a.res_len) == (b.quant_len, b.res_start, b.res_len)
        assert torch.equal(h_out, want.cpu()), "host decode step through the peer gather differs"
    pg.close()
def graph_replayed_gather(store, q_local, n_units, rank, world, want):
    """The exchange with its call counter on the device: plain calls, then two
    calls captured in a CUDA graph and replayed (a captured descriptor is frozen,
    the kernel advances the epoch and alternates the buffers itself)."""
    from intel_kivi_hybrid_b200.parallel import PeerGather
    pg = PeerGather(n_units, n_rep, D, torch.float32, rank, world, device_epoch=True)
    for i in range(3):
        store.attention_gather(q_local, pg.descriptor(), torch.float32, n_rep, num_splits=3)
        torch.cuda.synchronize()
        assert torch.equal(pg.gathered(), want), "device-epoch gather differs"
        assert pg.epoch == i + 1
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            store.attention_gather(q_local, pg.descriptor(), torch.float32, n_rep, num_splits=3)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(2):
            store.attention_gather(q_local, pg.descriptor(), torch.float32, n_rep, num_splits=3)
    for rep in range(3):
        pg.gathered().zero_()                           # the replay's second call rewrites this half
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(pg.gathered(), want), "graph-replayed gather differs"
        assert pg.epoch == 5 + 2 * (rep + 1)
    assert cabi.device_fault() == 0
    pg.close()
if world == 1:
    q_all = q.to(dev).reshape(B * Hkv, n_rep, D)     # (the store has taken two more tokens above: its own answer is the reference)
    graph_replayed_gather(st, q_all, B * Hkv, 0, 1, st.attention(q_all, n_rep=n_rep, num_splits=3, out_dtype=torch.float32))
else:
    u_per = B * Hkv // world
    graph_replayed_gather(sharded._stores[0], q.to(dev).reshape(B * Hkv, n_rep, D)[rank * u_per:(rank + 1) * u_per].contiguous(),
                          B * Hkv, rank, world, out_1.reshape(B * Hkv, n_rep, D))
    peer = KiviCache(num_layers=1, head_dim=D, device=dev, shard=(rank, world), gather="peer")
    peer.add_tokens(((K[:, :, :T - 3].to(dev), V[:, :, :T - 3].to(dev)),))
    peer.add_tokens(((K.to(dev), V.to(dev)),))
    for _ in range(3):
        out_p = peer.decode_attention(0, q.to(dev), out_dtype=torch.float32, num_splits=3)
        torch.cuda.synchronize()
        assert torch.equal(out_p, out_1), "peer-gather output differs from the single-GPU output"
    peer.close()
if world > 1:
    # the sequence sharded instead of the units: every rank holds all units and its share of the token groups
    seq = KiviCache(num_layers=1, head_dim=D, device=dev, shard=(rank, world), shard_mode="tokens")
    seq.add_tokens(((K[:, :, :T - 3].to(dev), V[:, :, :T - 3].to(dev)),))
    seq.add_tokens(((K.to(dev), V.to(dev)),))
    assert seq._quant_token_count[0] == single._quant_token_count[0] and seq._stores[0].quant_len < single._quant_token_count[0]
    out_t = seq.decode_attention(0, q.to(dev), out_dtype=torch.float32)
    torch.cuda.synchronize()
    err_t = ((out_t - out_1).abs().amax(-1) / out_1.abs().amax(-1)).max().item()
    assert err_t < 2e-3, err_t
assert cabi.device_fault() == 0
dist.barrier()
torch.cuda.synchronize()
dist.destroy_process_group()
print("ok", rank, err)
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_cache_equals_single_gpu(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29655", WORLD_SIZE="2",
               NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append("timeout")
    assert all(p.returncode == 0 for p in procs), outs
    assert all("ok" in o for o in outs), outs


@pytest.mark.skipif(torch.cuda.device_count() < 1, reason="needs a GPU")
def test_peer_gather_kernel_world_of_one(tmp_path):
    script = tmp_path / "worker1.py"
    script.write_text(_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29657", WORLD_SIZE="1", RANK="0")
    p = subprocess.run([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=240)
    assert p.returncode == 0 and "ok" in p.stdout, p.stdout


def test_peer_wait_that_runs_out_is_reported_and_can_be_cleared():
    """A bounded device-side wait seen to expire, without any fault: the gather
    descriptor names a second rank whose buffer and flag array are plain local
    allocations that nobody ever writes, and the wait is limited to about a
    millisecond.  The kernel must return, bit 1 of the fault word must be set,
    this rank's rows must be in both buffers, KiviCache must report the fault,
    and the word must be clearable."""
    import time
    from intel_kivi_hybrid_b200 import cabi
    from kivi_cuda import KiviCache
    from oracle import kivi_oracle as ko
    B, Hkv, n_rep, D, T, nq = 1, 4, 4, 128, 300, 256
    U = B * Hkv
    K = ko.make_keys(B, Hkv, T, D, 9).to(torch.bfloat16).reshape(U, T, D).cuda()
    V = ko.make_values(B, Hkv, T, D, 9).to(torch.bfloat16).reshape(U, T, D).cuda()
    q = ko.make_queries(B, Hkv * n_rep, D, 9).to(torch.bfloat16).reshape(U, n_rep, D).cuda()
    st = cabi.LayerStore(U, D, 32, 128, nq, torch.bfloat16, "cuda")
    cabi.load_state(st, K, V, nq)
    ref = st.attention(q, n_rep=n_rep, num_splits=2, out_dtype=torch.float32)
    bufs = [torch.zeros(2 * U, n_rep, D, device="cuda") for _ in range(2)]
    flags = [torch.zeros(cabi.PEER_MAX_WORLD, dtype=torch.int32, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    assert cabi.device_fault() == 0

    def expire(epoch):
        d = cabi.PeerGatherDesc()
        d.rank, d.world, d.unit_offset, d.epoch, d.wait, d.spin_limit = 0, 2, 0, epoch, 1, 5000
        for r in range(2):
            d.out_ptrs[r], d.flag_ptrs[r] = bufs[r].data_ptr(), flags[r].data_ptr()
        t0 = time.time()
        st.attention_gather(q, d, torch.float32, n_rep, num_splits=2)
        torch.cuda.synchronize()
        return time.time() - t0

    took = expire(1)
    assert took < 1.0, f"the bounded wait took {took:.2f} s"
    assert cabi.device_fault() == 2
    for b in bufs:                                   # this rank's rows reached both ranks' buffers
        assert torch.equal(b[:U], ref) and not b[U:].any()
    assert flags[0].tolist()[:2] == [1, 0] and flags[1].tolist()[:2] == [1, 0]
    cabi.device_fault_clear()
    assert cabi.device_fault() == 0
    expire(2)
    cache = KiviCache(num_layers=1, head_dim=D)
    with pytest.raises(RuntimeError, match="peer rank did not publish"):
        cache.check_device_fault()
    assert cabi.device_fault() == 0                  # reported once, then cleared
    out = st.attention(q, n_rep=n_rep, num_splits=2, out_dtype=torch.float32)
    assert torch.equal(out, ref)                     # the context is as usable as before


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-3), (torch.float32, 1e-5)])
def test_sequence_sharded_cache_on_one_gpu(dtype, tol):
    """shard_mode="tokens" with the three ranks of a world held in one process:
    every token group is kept by exactly one rank, the rings stay replicated, and
    the folded partial attentions equal an unsharded cache's output through a
    prefill, single-token steps across several flushes, and a multi-token chunk."""
    from intel_kivi_hybrid_b200 import cabi
    from kivi_cuda import KiviCache
    from oracle import kivi_oracle as ko
    B, Hkv, n_rep, D, G, R, world = 1, 2, 4, 128, 32, 128, 3
    T0, steps = 500, 75
    T = T0 + steps + 40
    K = ko.make_keys(B, Hkv, T, D, 51).to(dtype).cuda()
    V = ko.make_values(B, Hkv, T, D, 51).to(dtype).cuda()
    full = KiviCache(num_layers=1, head_dim=D, device="cuda")
    ranks = [KiviCache(num_layers=1, head_dim=D, device="cuda", shard=(r, world), shard_mode="tokens") for r in range(world)]

    def feed(t):
        for c in [full] + ranks:
            c.add_tokens(((K[:, :, :t], V[:, :, :t]),))

    def check(t):
        q = ko.make_queries(B, Hkv * n_rep, D, seed=t).to(dtype).cuda()
        qu = q.reshape(B * Hkv, n_rep, D).contiguous()
        parts = torch.stack([c.token_shard_partial(0, qu, n_rep) for c in ranks])
        merged = cabi.merge_token_shards(parts).reshape(B, Hkv * n_rep, D)
        ref = full.decode_attention(0, q, out_dtype=torch.float32)
        err = float(((merged - ref).abs().amax(-1) / ref.abs().amax(-1)).max())
        assert err < tol, (t, err)
        kept = [c._stores[0].quant_len for c in ranks]
        assert sum(kept) == full._quant_token_count[0] == ranks[0]._quant_token_count[0]
        assert max(kept) - min(kept) <= 2 * G                       # balanced
        for c in ranks:                                             # replicated ring, same window
            assert torch.equal(c.res_keys[0], full.res_keys[0])
        return err

    feed(T0); check(T0)
    worst = 0.0
    for t in range(T0 + 1, T0 + steps + 1):
        feed(t)
        worst = max(worst, check(t))
    feed(T); check(T)                                               # 40 tokens at once on a non-empty cache
    assert full.total_flushes == ranks[1].total_flushes > (T0 - R) // G + 2
    print(f"[sequence sharding, {dtype}] worst error vs the unsharded cache {worst:.2e}")
    # the oracle agrees with the folded result as well
    q = ko.make_queries(B, Hkv * n_rep, D, seed=9).to(dtype)
    parts = torch.stack([c.token_shard_partial(0, q.cuda().reshape(B * Hkv, n_rep, D).contiguous(), n_rep) for c in ranks])
    got = cabi.merge_token_shards(parts).reshape(B, Hkv * n_rep, D).cpu()
    ref = ko.kivi_decode_attention(q, K.cpu(), V.cpu(), full._quant_token_count[0], G, "half_away", dtype=torch.float64).float()
    assert float(((got - ref).abs().amax(-1) / ref.abs().amax(-1)).max()) < tol
