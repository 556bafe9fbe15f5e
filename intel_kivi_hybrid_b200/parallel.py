"""Sharding of the (batch, kv_head) units over the GPUs of one node.

Every unit is independent end to end (quantize, flush, attention), so rank r
of `world` permanently owns a contiguous run of units and no KV ever crosses
NVLink.  The one exchange per layer-step is an all-gather of the attention
outputs [units, n_rep, D] (the reference is single-device: nothing to cite).
Works on any torch.distributed backend: NCCL on GPUs, gloo in the CPU tests.

`PeerGather` is the fused form of that exchange on GPUs: the attention's last
kernel stores every output row into all ranks' gathered buffers through
peer-mapped memory and the ranks synchronise through flags in the same memory,
so no separate collective is launched.
"""
from typing import Tuple

import torch

__all__ = ["unit_partition", "all_gather_units", "PeerGather", "merge_token_shards", "TokenShardPlan"]


def unit_partition(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """[u0, u1) of rank `rank`: contiguous, sizes differ by at most one, the
    first n_units % world ranks hold the extra unit."""
    assert 0 <= rank < world and n_units >= 0
    base, extra = divmod(n_units, world)
    u0 = rank * base + min(rank, extra)
    return u0, u0 + base + (1 if rank < extra else 0)


def all_gather_units(local: torch.Tensor, n_units: int, rank: int, world: int, group=None) -> torch.Tensor:
    """local [u1-u0, ...] of every rank -> [n_units, ...] on every rank, in unit
    order.  Equal shards use one all_gather_into_tensor; ragged shards pad to
    the largest shard first."""
    import torch.distributed as dist
    if world == 1:
        return local
    sizes = [unit_partition(n_units, r, world) for r in range(world)]
    biggest = max(b - a for a, b in sizes)
    tail = local.shape[1:]
    if all(b - a == biggest for a, b in sizes):
        out = torch.empty((n_units,) + tuple(tail), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest,) + tuple(tail), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    buf = torch.empty((world * biggest,) + tuple(tail), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    return torch.cat([buf[r * biggest: r * biggest + (b - a)] for r, (a, b) in enumerate(sizes)], dim=0)


class TokenShardPlan:
    """Which rank keeps which token group when the *sequence* is sharded (every
    rank holds all units but only its share of each unit's quantized groups; the
    residual ring is replicated).  Attention is a sum over tokens, so any
    assignment that gives every group to exactly one rank is correct; this one
    keeps the ranks balanced as the sequence grows:

    * a bulk flush of ``f`` groups at once (prefill) is cut into ``world``
      contiguous runs, rank r taking run r (``unit_partition`` of the f groups);
    * groups flushed one at a time (decode) go round robin, group number g to
      rank ``g % world``.

    Pure arithmetic on the global group count: every rank computes the same plan
    without talking to the others (the reference has no counterpart: it is
    single-device and keeps the whole history dequantized,
    cache/manager.py:100-117)."""

    def __init__(self, rank: int, world: int):
        assert 0 <= rank < world
        self.rank, self.world = rank, world

    def bulk_run(self, n_groups: int) -> Tuple[int, int]:
        """[g0, g1) of a bulk flush of n_groups groups that this rank keeps."""
        return unit_partition(n_groups, self.rank, self.world)

    def owner(self, global_group: int) -> int:
        """Rank that keeps a group flushed on its own (decode)."""
        return global_group % self.world

    def owns(self, global_group: int) -> bool:
        return self.owner(global_group) == self.rank

    @property
    def serves_ring(self) -> bool:
        """The replicated ring is attended by one rank only (rank 0)."""
        return self.rank == 0


def merge_token_shards(outs: torch.Tensor, lses: torch.Tensor) -> torch.Tensor:
    """Combine attention outputs computed over disjoint token ranges of the same
    sequences (sequence sharding: every rank holds a slice of each unit's
    history and runs LayerStore.attention_lse on it).
    outs [n_shards, ..., D], lses [n_shards, ...] (natural-log sums of
    exponentials) -> [..., D] in fp32:  sum_i out_i * exp(lse_i - LSE)."""
    lses = lses.float()
    total = torch.logsumexp(lses, dim=0, keepdim=True)
    w = torch.exp(lses - total).unsqueeze(-1)
    return (outs.float() * w).sum(dim=0)


class PeerGather:
    """Gathered attention-output buffers of the ranks of one node, mapped into
    every rank (CUDA IPC through kivi_peer_alloc / kivi_peer_open), for
    LayerStore.attention_gather.  ``device_epoch=True`` keeps the call counter on
    the GPU: calls can then be captured in a CUDA graph and replayed.

    Each rank owns two gathered buffers [n_units * n_rep * D] (alternated by
    epoch parity, so a rank that runs one call ahead never overwrites what a
    slower rank's consumer is still reading) and one flag array.  Setup is
    collective over `group` (handles travel by all_gather_object); equal unit
    counts per rank are not required.
    """

    def __init__(self, n_units: int, n_rep: int, head_dim: int, dtype, rank: int, world: int, group=None,
                 device_epoch: bool = False):
        import torch.distributed as dist
        from . import cabi
        assert 1 <= world <= cabi.PEER_MAX_WORLD
        self._cabi, self.rank, self.world, self.dtype = cabi, rank, world, dtype
        self.n_units, self.n_rep, self.D = n_units, n_rep, head_dim
        self.u0, self.u1 = unit_partition(n_units, rank, world)
        esz = torch.empty((), dtype=dtype).element_size()
        self._buf_bytes = -(-n_units * n_rep * head_dim * esz // 256) * 256
        # one allocation per rank: [buffer 0 | buffer 1 | flags].  Every rank takes
        # part in every exchange below even after a local failure, so that all
        # ranks raise together instead of one of them leaving the others waiting.
        self._own_ptr, self._ptrs, handle, err = 0, [], None, None
        try:
            self._own_ptr, handle = cabi.peer_alloc(2 * self._buf_bytes + 256)
        except RuntimeError as exc:
            err = f"rank {rank}: {exc}"
        handles = [None] * world
        dist.all_gather_object(handles, (handle, err), group=group)
        if all(h is not None for h, _ in handles):
            try:
                for r in range(world):
                    self._ptrs.append(self._own_ptr if r == rank else cabi.peer_open(handles[r][0]))
            except RuntimeError as exc:
                err = f"rank {rank}: {exc}"
        errs = [None] * world
        dist.all_gather_object(errs, err, group=group)
        failed = [e for e in errs if e] + [e for _, e in handles if e]
        if failed:
            for r, p in enumerate(self._ptrs):
                if r != rank:
                    cabi.peer_close(p)
            dist.barrier(group=group)
            if self._own_ptr:
                cabi.peer_free(self._own_ptr)
            self._ptrs, self._own_ptr = [], 0
            raise RuntimeError("peer-gather setup failed: " + "; ".join(sorted(set(failed))))
        self.epoch = 0
        # device_epoch: the call counter lives on the GPU, so that a call can be
        # captured in a CUDA graph and replayed (a captured descriptor is frozen)
        self._epoch_dev = (torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
                           if device_epoch else None)
        dist.barrier(group=group)

    def descriptor(self, wait: bool = True, spin_limit: int = 0, wait_stats: torch.Tensor = None):
        """The kivi_peer_gather of the next call (advances the epoch).
        ``spin_limit``: bound of the wait for the other ranks in polls of about
        200 ns (0 = the library's default, about a second).  ``wait_stats``: an
        int64[2] device tensor the kernel adds its waiting time (ns) and 1 to."""
        c = self._cabi
        self.epoch += 1
        d = c.PeerGatherDesc()
        d.rank, d.world, d.unit_offset, d.epoch, d.wait = self.rank, self.world, self.u0, self.epoch, int(wait)
        d.spin_limit = int(spin_limit)
        d.wait_stats = wait_stats.data_ptr() if wait_stats is not None else None
        half = (self.epoch & 1) * self._buf_bytes
        if self._epoch_dev is not None:                 # the kernel picks the half from its own counter
            d.epoch_dev, d.alt_bytes, half = self._epoch_dev.data_ptr(), self._buf_bytes, 0
        for r in range(self.world):
            d.out_ptrs[r] = self._ptrs[r] + half
            d.flag_ptrs[r] = self._ptrs[r] + 2 * self._buf_bytes
        return d

    def gathered(self) -> torch.Tensor:
        """[n_units, n_rep, D] view of this rank's gathered buffer of the last
        call (valid once that call's kernels have completed on the stream; with a
        device-kept epoch the counter is read back, which synchronises)."""
        n = self.n_units * self.n_rep * self.D
        if self._epoch_dev is not None:
            self.epoch = int(self._epoch_dev.item())
        half = (self.epoch & 1) * self._buf_bytes
        device = torch.device("cuda", torch.cuda.current_device())
        return _tensor_from_ptr(self._own_ptr + half, n, self.dtype, device).view(self.n_units, self.n_rep, self.D)

    def close(self, group=None):
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=group)                       # nobody still writes into a peer
        for r, p in enumerate(self._ptrs):
            if r != self.rank and p:
                self._cabi.peer_close(p)
        dist.barrier(group=group)                       # every mapping is gone before the owner frees
        if self._own_ptr:
            self._cabi.peer_free(self._own_ptr)
        self._ptrs, self._own_ptr = [], 0


class _CudaArray:
    """__cuda_array_interface__ holder so that torch can view foreign device memory."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3}


def _tensor_from_ptr(ptr: int, n: int, dtype, device) -> torch.Tensor:
    if dtype == torch.bfloat16:          # no typestr for bf16: view 16-bit words
        return torch.as_tensor(_CudaArray(ptr, n, "<i2"), device=device).view(torch.bfloat16)
    return torch.as_tensor(_CudaArray(ptr, n, "<f4"), device=device)
