"""CPU-only checks of the host side: the C-ABI library loads and exports every
symbol the header declares, the flush arithmetic equals the reference policy,
unit sharding and its gather (gloo, world size 2), config sniffing, sampling,
and the Python surface of the drop-in API.  No kernel is launched here."""
import ctypes
import os
import re
import subprocess
import sys
import types

import pytest
import torch

from oracle import kivi_oracle as ko

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from intel_kivi_hybrid_b200 import _build, cabi
    hdr = open(os.path.join(ROOT, "include", "kivi_cuda.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(kivi_[a-z0-9_]+)\s*\(", hdr))
    assert {"kivi_quantize_keys_per_channel", "kivi_cache_update", "kivi_decode_attention"} <= declared
    lib = ctypes.CDLL(_build.LIB)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/kivi_cuda.h but not exported"
    assert declared == set(cabi.SIGNATURES), "ctypes binding and header list different entry points"
    assert cabi.lib.kivi_version() >= 100


def test_cache_plan_equals_reference_flush_policy():
    from intel_kivi_hybrid_b200 import cabi
    for G, R in ((4, 8), (32, 128), (16, 16), (32, 100), (64, 64)):
        for ql in (0, G, 5 * G):
            for rl in (0, 1, R - G, R - 1):
                for n in (1, 2, G - 1, G, R, 3 * R + 5, 8192):
                    f, q2, r2 = ko.flush_schedule(ql, rl, n, G, R)
                    assert cabi.cache_plan(ql, rl, n, G, R) == (f, q2, r2)
    assert cabi.cache_plan(0, 0, 512, 32, 128) == (13, 416, 96)     # 512-token prefill of config 0
    with pytest.raises(RuntimeError, match="group_size"):
        cabi.cache_plan(0, 0, 1, 64, 32)


def test_host_side_validation_needs_no_gpu():
    from intel_kivi_hybrid_b200 import cabi
    # null pointers / bad sizes are rejected on the host before any CUDA call
    rc = cabi.lib.kivi_quantize_keys_per_channel(None, 0, None, None, None, 4, 32, 0, None)
    assert rc == 1 and b"null" in cabi.lib.kivi_last_error()
    rc = cabi.lib.kivi_dequantize_keys_per_channel(None, None, None, None, 4, 6, None)
    assert rc == 1
    assert cabi.lib.kivi_decode_attention_workspace(512, 4, 128, 0) == 512 * (128 + 8) * 4 * 130 * 4
    assert cabi.lib.kivi_decode_attention_max_splits() == 128


def test_unit_partition_covers_every_unit_once():
    from intel_kivi_hybrid_b200.parallel import unit_partition
    for n in (1, 7, 32, 512, 513):
        for world in (1, 2, 4, 8):
            parts = [unit_partition(n, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1


_GLOO_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from intel_kivi_hybrid_b200.parallel import all_gather_units, unit_partition
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
for n_units in (8, 7):                       # equal and ragged shards
    full = torch.arange(n_units * 3 * 4, dtype=torch.float32).reshape(n_units, 3, 4)
    u0, u1 = unit_partition(n_units, rank, world)
    got = all_gather_units(full[u0:u1].clone(), n_units, rank, world)
    assert torch.equal(got, full), (rank, n_units)
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
'''


def test_all_gather_units_gloo_world2(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("ok" in o for o in outs)


_PEER_FAIL_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from intel_kivi_hybrid_b200.parallel import PeerGather
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
try:
    PeerGather(8, 4, 128, torch.bfloat16, rank, world)      # no GPU here: the allocation fails on every rank
    print("no error", rank)
except RuntimeError as exc:
    assert "peer-gather setup failed" in str(exc) and "rank 0" in str(exc) and "rank 1" in str(exc), exc
    print("ok", rank)
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the failure path of a box without GPUs")
def test_peer_gather_setup_fails_on_all_ranks_together(tmp_path):
    """A rank whose buffer cannot be allocated still takes part in every exchange
    of the setup, so all ranks raise the same error and none is left waiting."""
    script = tmp_path / "worker.py"
    script.write_text(_PEER_FAIL_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29643", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("ok" in o for o in outs), outs


def test_peer_gather_descriptor_alternates_buffers():
    from intel_kivi_hybrid_b200 import cabi
    from intel_kivi_hybrid_b200.parallel import PeerGather
    pg = PeerGather.__new__(PeerGather)          # no allocation: only the descriptor arithmetic
    pg._cabi, pg.rank, pg.world, pg.u0, pg.epoch = cabi, 1, 2, 4, 0
    pg._buf_bytes, pg._ptrs, pg._epoch_dev = 4096, [0x10000, 0x20000], None
    d1, d2, d3 = pg.descriptor(), pg.descriptor(wait=False), pg.descriptor()
    assert (d1.epoch, d2.epoch, d3.epoch) == (1, 2, 3) and (d1.wait, d2.wait) == (1, 0)
    assert (d1.rank, d1.world, d1.unit_offset) == (1, 2, 4)
    assert [d1.out_ptrs[r] for r in range(2)] == [0x10000 + 4096, 0x20000 + 4096]      # odd epoch: second half
    assert [d2.out_ptrs[r] for r in range(2)] == [0x10000, 0x20000]
    assert [d3.out_ptrs[r] for r in range(2)] == [d1.out_ptrs[r] for r in range(2)]
    assert [d1.flag_ptrs[r] for r in range(2)] == [0x10000 + 8192, 0x20000 + 8192]
    assert d1.out_ptrs[2] is None and d1.epoch_dev is None
    # call counter on the device: the descriptor names the first buffer and the distance to the second
    pg._epoch_dev = types.SimpleNamespace(data_ptr=lambda: 0x30000)
    d4 = pg.descriptor()
    assert (d4.epoch_dev, d4.alt_bytes) == (0x30000, 4096)
    assert [d4.out_ptrs[r] for r in range(2)] == [0x10000, 0x20000]


def test_detect_model_config_families():
    from intel_kivi_hybrid_b200.config.model_config import detect_model_config
    mk = lambda **kw: types.SimpleNamespace(config=types.SimpleNamespace(**kw))
    assert detect_model_config(mk(n_layer=12, n_head=12, n_embd=768)) == \
        {"num_layers": 12, "num_kv_heads": 12, "head_dim": 64}                      # GPT-2
    assert detect_model_config(mk(num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                                  hidden_size=4096)) == {"num_layers": 32, "num_kv_heads": 8, "head_dim": 128}  # Llama-3-8B
    assert detect_model_config(mk(num_hidden_layers=2, num_attention_heads=4, hidden_size=64, head_dim=32))["head_dim"] == 32
    with pytest.raises(ValueError, match="num_layers"):
        detect_model_config(mk(n_head=2, n_embd=8))
    with pytest.raises(ValueError, match="head_dim"):
        detect_model_config(mk(n_layer=2, n_head=2))


def test_sample_token():
    from intel_kivi_hybrid_b200.generation.sampling import sample_token
    logits = torch.tensor([[0.1, 3.0, -1.0, 2.0], [5.0, 0.0, 0.0, 0.0]])
    assert sample_token(logits, 1.0, None, False).tolist() == [[1], [0]]
    torch.manual_seed(0)
    for _ in range(20):
        t = sample_token(logits.clone(), 0.7, 2, True)
        assert t.shape == (2, 1) and t[0, 0].item() in (1, 3) and t[1, 0].item() in (0, 1, 2, 3)


def test_drop_in_surface():
    import kivi_cuda
    import kivi_sycl
    from kivi_sycl import KiviCache, generate, __version__
    assert __version__ == "0.1.0" and kivi_cuda.KiviCache is KiviCache and callable(generate)
    with pytest.raises(AssertionError, match="divisible by group_size"):
        KiviCache(2, 48, group_size=32)
    with pytest.raises(AssertionError, match="must not exceed residual_length"):
        KiviCache(2, 64, group_size=64, residual_length=32)
    with pytest.raises(AssertionError, match=">= 4 and divisible by 4"):
        KiviCache(2, 64, group_size=2)
    c = KiviCache(num_layers=3, head_dim=64, num_kv_heads=2, device="cuda", group_size=32, residual_length=128)
    assert (c.G, c.R, c.num_layers, c.batch_size, c.total_flushes) == (32, 128, 3, None, 0)
    assert c._quant_token_count == [0, 0, 0] and c.res_keys == [None, None, None]
    assert repr(c) == "KiviCache(layers=3, head_dim=64, G=32, R=128, device='cuda')"
    assert c.get_stats()["compression"] == 0
    # the twelve operators + KiviEvent, with the reference's keyword names (pybind_module.cpp:18-81)
    from kivi_sycl import _C
    ops = ["quantize_keys", "quantize_values", "dequantize_keys", "dequantize_values",
           "quant_dequant_roundtrip_keys", "quant_dequant_roundtrip_values"]
    for op in ops:
        assert callable(getattr(_C, op)) and callable(getattr(_C, op + "_async"))
    assert hasattr(_C.KiviEvent, "wait")
    doc = _C.quantize_values.__doc__
    for kw in ("input", "output", "scales", "zeros", "head_dim", "group_size"):
        assert kw + ":" in doc
    x = torch.zeros(64)
    with pytest.raises(RuntimeError, match="must be on cuda"):
        _C.quant_dequant_roundtrip_keys(input=x, output=torch.zeros(64), group_size=32)


def test_merge_token_shards_equals_attention_over_the_whole_sequence():
    """Outputs over disjoint token ranges + their log-sum-exps combine into the
    attention over the union (the host side of sequence sharding)."""
    from intel_kivi_hybrid_b200.parallel import merge_token_shards
    torch.manual_seed(3)
    U, H, D, T = 3, 4, 16, 50
    q = torch.randn(U, H, D, dtype=torch.float64)
    k = torch.randn(U, T, D, dtype=torch.float64)
    v = torch.randn(U, T, D, dtype=torch.float64)
    s = torch.einsum("uhd,utd->uht", q, k) * D ** -0.5
    whole = torch.einsum("uht,utd->uhd", torch.softmax(s, -1), v)
    outs, lses = [], []
    for a, b in ((0, 7), (7, 31), (31, T)):
        outs.append(torch.einsum("uht,utd->uhd", torch.softmax(s[..., a:b], -1), v[:, a:b]))
        lses.append(torch.logsumexp(s[..., a:b], -1))
    got = merge_token_shards(torch.stack(outs).float(), torch.stack(lses).float())
    assert got.dtype == torch.float32 and torch.allclose(got.double(), whole, atol=1e-6)


def test_operands_on_different_devices_are_refused_before_any_launch():
    """A kernel runs on one GPU and must not be handed another GPU's pointers:
    the binding compares the devices of all tensors of a call on the host.
    Stand-ins with a .device are enough: nothing is launched."""
    from intel_kivi_hybrid_b200 import cabi

    class T:
        is_cuda = True

        def __init__(self, device):
            self.device = torch.device(device)

        def is_contiguous(self):
            return True

    cabi._dev(T("cuda:0"), T("cuda:0"))
    with pytest.raises(RuntimeError, match="same device"):
        cabi._dev(T("cuda:0"), T("cuda:0"), T("cuda:1"))
    with pytest.raises(RuntimeError, match="same device"):
        cabi.quantize_keys(T("cuda:0"), T("cuda:1"), T("cuda:0"), T("cuda:0"), 32)


def test_peer_gather_descriptor_layout_matches_the_header():
    """struct kivi_peer_gather as ctypes sees it: the C compiler's layout of the
    header's fields (two ints, 2 x 8 pointers, int64, four 32-bit words, two pointers' worth at the end)."""
    from intel_kivi_hybrid_b200 import cabi
    d = cabi.PeerGatherDesc
    assert d.out_ptrs.offset == 8 and d.flag_ptrs.offset == 8 + 8 * cabi.PEER_MAX_WORLD
    assert d.unit_offset.offset == 8 + 16 * cabi.PEER_MAX_WORLD
    assert (d.epoch.offset, d.wait.offset, d.spin_limit.offset) == (d.unit_offset.offset + 8, d.unit_offset.offset + 12,
                                                                    d.unit_offset.offset + 16)
    import ctypes
    assert d.wait_stats.offset == d.unit_offset.offset + 24
    assert (d.epoch_dev.offset, d.alt_bytes.offset) == (d.unit_offset.offset + 32, d.unit_offset.offset + 40)
    assert ctypes.sizeof(d) == d.unit_offset.offset + 48


def test_attention_split_plan_is_pinned():
    """kivi_decode_attention_plan is host arithmetic: pin what it chooses for the
    benchmark shapes on a 148-SM GPU holding 3 CTAs of the tensor-core kernel per
    SM (units, quantized tokens, ring tokens) -> (tensor cores, pieces, ring CTAs)."""
    from intel_kivi_hybrid_b200 import cabi
    plan = lambda *a, **k: cabi.attention_plan(*a, sms=148, ctas_per_sm=3, **k)
    assert plan(512, 32640, 128) == (True, 4, 1)          # batch 64, 32k context: several waves of ~250-group CTAs
    assert plan(128, 3968, 128) == (True, 2, 1)           # batch 16, 4k context: 256 CTAs, at most two per SM
    assert plan(32, 131072, 128) == (True, 13, 1)         # batch 4, 128k context: 13*32 CTAs fill the 444 slots once
    assert plan(64, 32640, 128) == (True, 6, 1)           # 1/8 of the batch-64 workload (8-GPU shard): 384 CTAs at once
    assert plan(16, 65536, 128) == (True, 27, 1)
    assert plan(4, 131072, 128) == (True, 64, 1)          # few units, long context: many pieces, folded by a CTA per row
    assert plan(512, 32640, 128, num_splits=7) == (True, 7, 1)            # a caller-fixed count is taken as given
    assert plan(512, 32640, 0)[2] == 0 and plan(512, 32640, 1000)[2] == 8  # ring CTAs: none / capped at 8
    assert plan(4, 64, 0, n_rep=8) == (True, 1, 0)        # 8 heads per KV head: two head blocks per unit on the tensor cores
    assert plan(4, 64, 0, n_rep=9)[0] is False            # more than 8: CUDA-core kernel
    assert plan(12, 512, 96, head_dim=64, q_dtype=cabi.F32)[0] is False
    with pytest.raises(RuntimeError, match="tensor-core path"):
        plan(12, 512, 96, head_dim=64, path=cabi.ATTN_MMA)


def test_attention_split_plan_stays_in_range_and_fills_the_machine():
    """Whatever the shape, the planner returns between 1 and min(groups, 128) pieces,
    never leaves most of the GPU idle when there are groups to hand out, and never
    cuts a big batch of short contexts into crumbs."""
    from intel_kivi_hybrid_b200 import cabi
    plan = lambda u, t: cabi.attention_plan(u, t, 128, sms=148, ctas_per_sm=3)[1]
    for units in (1, 2, 3, 5, 8, 16, 31, 64, 100, 128, 222, 256, 500, 512, 1024, 4096):
        for tokens in (32, 64, 512, 4096, 32768, 131072):
            s = plan(units, tokens)
            groups = tokens // 32
            assert 1 <= s <= min(groups, 128), (units, tokens, s)
            if units * groups >= 4 * 148:                        # enough work for every SM
                assert units * s >= 48, (units, tokens, s)       # ... then at least 48 CTAs are started
            if units >= 444 and groups <= 128:
                assert s <= 2, (units, tokens, s)                # a full wave of short units: one or two pieces each
    assert plan(1, 32) == 1 and plan(4096, 32) == 1


def test_token_shard_plan_gives_every_group_to_one_rank():
    from intel_kivi_hybrid_b200.parallel import TokenShardPlan
    for world in (1, 2, 3, 8):
        plans = [TokenShardPlan(r, world) for r in range(world)]
        for f in (0, 1, 5, 17, 64):                                   # a bulk flush: contiguous runs covering 0..f
            runs = [p.bulk_run(f) for p in plans]
            assert runs[0][0] == 0 and runs[-1][1] == f
            assert all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
            assert max(b - a for a, b in runs) - min(b - a for a, b in runs) <= 1
        for g in range(40):                                           # single groups: exactly one owner
            assert sum(p.owns(g) for p in plans) == 1
        assert sum(p.serves_ring for p in plans) == 1
