"""CPU oracle for the KIVI 2-bit KV-cache path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: it is the checker that
the parity tests, the smoke check and the CPU-baseline leg of the benchmark
compare the CUDA kernels against.  Every function is a restatement, in torch
CPU ops, of arithmetic the reference project writes down itself; the citation
beside each function is ``path:line`` inside that project.

Parity status
-------------
* group quantize / dequantize / round-trip: PINNED.  The restatement is checked
  bit-for-bit against the reference's own torch mirror
  (examples/cpu_sim.py:37-43, tests/unit/test_manager_bookkeeping.py:36-48,
  tests/integration/test_roundtrip_kernels.py:21-27) through the vectors in
  tests/golden/ (made by tests/golden/make_golden.py by importing the
  reference), and against the known answers the reference tests hold
  ([1,2,3,4] -> byte 228, constant 5.0, codes in [0,3]).
* residual / flush state machine: PINNED against the reference's own
  ``KiviCache`` driven by its ``FakeModel`` (golden vectors, same script).
* decode attention: the formula is tests/integration/test_attention_fix.py:40-43
  applied to ``history || residual`` (cache/manager.py:263-286).  The reference
  has no attention kernel and pins attention only through a cosine>0.85 check,
  so for the 1e-5 / 2e-3 tolerances this part is "parity unpinned": it is this
  build's restatement of the reference's formula, pinned only to the golden
  vector generated from that test's seed-42 inputs.

Two rounding conventions exist in the reference and both are provided:
``half_even`` is what the reference's torch mirror does (torch.round,
examples/cpu_sim.py:42) and ``half_away`` is what its device kernel does
(sycl::round, src/csrc/kernels/internal/quant_tile.hpp:64,85).  They differ only
where (x-min)/scale is exactly 0.5 or 2.5; ``tie_mask`` marks those elements.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

__all__ = [
    "group_params", "group_codes", "pack_codes", "unpack_codes",
    "quantize_groups", "dequantize_groups", "roundtrip_groups", "tie_mask",
    "quantize_keys", "quantize_values", "dequantize_keys", "dequantize_values",
    "flush_schedule", "OracleCache", "attention", "kivi_decode_attention",
    "make_keys", "make_values", "make_queries", "algorithmic_bytes_attention",
    "algorithmic_bytes_quantize",
]


# --------------------------------------------------------------------------
# Per-group arithmetic
# --------------------------------------------------------------------------

def group_params(flat: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """min and scale of each row of ``flat`` ([num_groups, G], fp32).

    ``scale = (max - min) / 3.0f + 1e-10f``, ``zero = min``
    (src/csrc/kernels/quantize_kernels.cpp:46-48; examples/cpu_sim.py:39-41).
    """
    assert flat.dtype == torch.float32 and flat.dim() == 2
    mn = flat.min(dim=1, keepdim=True).values
    mx = flat.max(dim=1, keepdim=True).values
    scale = (mx - mn) / 3.0 + 1e-10
    return mn, scale


def _round(t: torch.Tensor, rounding: str) -> torch.Tensor:
    if rounding == "half_even":          # torch.round, examples/cpu_sim.py:42
        return torch.round(t)
    if rounding == "half_away":          # sycl::round, quant_tile.hpp:64
        # t >= 0 always here (t = (x - min) / scale), so away-from-zero is
        # floor(t + 0.5) evaluated without a second rounding: compare the
        # fractional part instead of adding 0.5 in floating point.
        fl = torch.floor(t)
        return torch.where(t - fl >= 0.5, fl + 1.0, fl)
    raise ValueError(rounding)


def group_codes(flat: torch.Tensor, rounding: str = "half_even"
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """codes (fp32 values in {0,1,2,3}), scale, min for each row of ``flat``.

    ``q = clamp(round((x - min) / scale), 0, 3)``
    (quant_tile.hpp:61-66; examples/cpu_sim.py:42).
    """
    mn, scale = group_params(flat)
    q = torch.clamp(_round((flat - mn) / scale, rounding), 0.0, 3.0)
    return q, scale, mn


def tie_mask(flat: torch.Tensor) -> torch.Tensor:
    """True where (x-min)/scale is exactly 0.5 or 2.5, i.e. where the two
    rounding conventions of the reference give different codes."""
    mn, scale = group_params(flat)
    t = (flat - mn) / scale
    return (t == 0.5) | (t == 2.5)


def pack_codes(q: torch.Tensor) -> torch.Tensor:
    """``byte = q0 | q1<<2 | q2<<4 | q3<<6`` over consecutive runs of four
    codes (quant_tile.hpp:61-68).  ``q``: [..., 4k] integral values."""
    qi = q.to(torch.int32).reshape(*q.shape[:-1], q.shape[-1] // 4, 4)
    b = qi[..., 0] | (qi[..., 1] << 2) | (qi[..., 2] << 4) | (qi[..., 3] << 6)
    return b.to(torch.uint8)


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_codes` (dequantize_kernels.cpp:23-25)."""
    p = packed.to(torch.int32).unsqueeze(-1)
    sh = torch.tensor([0, 2, 4, 6], dtype=torch.int32)
    return ((p >> sh) & 3).reshape(*packed.shape[:-1], packed.shape[-1] * 4)


def quantize_groups(x: torch.Tensor, group_size: int,
                    rounding: str = "half_even") -> Dict[str, torch.Tensor]:
    """Quantize the flat view of ``x`` in runs of ``group_size``.

    Both reference kernels (keys per channel, values per token) reduce over
    contiguous runs of ``group_size`` elements of the flat input
    (quantize_kernels.cpp:42,93; test_manager_bookkeeping.py:39-41), so one
    flat function is the oracle for both.  Returns packed [N/4] u8,
    scales/zeros [N/G] fp32, codes [N] u8.
    """
    flat = x.detach().to(torch.float32).reshape(-1, group_size)
    q, scale, mn = group_codes(flat, rounding)
    return {
        "packed": pack_codes(q).reshape(-1),
        "scales": scale.reshape(-1).clone(),
        "zeros": mn.reshape(-1).clone(),
        "codes": q.to(torch.uint8).reshape(-1),
    }


def dequantize_groups(packed: torch.Tensor, scales: torch.Tensor,
                      zeros: torch.Tensor, group_size: int) -> torch.Tensor:
    """``out = float(code) * scale + zero`` with a separate multiply and add
    (dequantize_kernels.cpp:23-27; examples/cpu_sim.py:43).  Flat fp32 out."""
    codes = unpack_codes(packed.reshape(-1, group_size // 4)).to(torch.float32)
    return (codes * scales.reshape(-1, 1) + zeros.reshape(-1, 1)).reshape(-1)


def roundtrip_groups(x: torch.Tensor, group_size: int,
                     rounding: str = "half_even") -> torch.Tensor:
    """Fused quantize->dequantize (roundtrip_kernels.cpp:27-33,
    quant_tile.hpp:74-91; examples/cpu_sim.py:37-43).  Same shape as ``x``."""
    flat = x.detach().to(torch.float32).reshape(-1, group_size)
    q, scale, mn = group_codes(flat, rounding)
    return (q * scale + mn).reshape(x.shape)


# Operator-shaped wrappers (layouts of README.md:120-136) -----------------

def quantize_keys(k_bhds: torch.Tensor, group_size: int, rounding="half_even"):
    """keys, already transposed to [B,H,D,S]: groups run along S
    (quantize_kernels.hpp:33-42)."""
    B, H, D, S = k_bhds.shape
    r = quantize_groups(k_bhds.contiguous(), group_size, rounding)
    return (r["packed"].reshape(B, H, D, S // 4),
            r["scales"].reshape(B, H, D, S // group_size),
            r["zeros"].reshape(B, H, D, S // group_size))


def quantize_values(v_bhsd: torch.Tensor, group_size: int, rounding="half_even"):
    """values [B,H,S,D]: groups run along D (quantize_kernels.hpp:55-60)."""
    B, H, S, D = v_bhsd.shape
    r = quantize_groups(v_bhsd.contiguous(), group_size, rounding)
    return (r["packed"].reshape(B, H, S, D // 4),
            r["scales"].reshape(B, H, S, D // group_size),
            r["zeros"].reshape(B, H, S, D // group_size))


def dequantize_keys(packed, scales, zeros, group_size):
    B, H, D, S4 = packed.shape
    return dequantize_groups(packed, scales, zeros, group_size).reshape(B, H, D, S4 * 4)


def dequantize_values(packed, scales, zeros, group_size):
    B, H, S, D4 = packed.shape
    return dequantize_groups(packed, scales, zeros, group_size).reshape(B, H, S, D4 * 4)


# --------------------------------------------------------------------------
# Residual window / flush policy
# --------------------------------------------------------------------------

def flush_schedule(quantized: int, residual: int, new: int, G: int, R: int
                   ) -> Tuple[int, int, int]:
    """State after appending ``new`` tokens: (flushes, quantized, residual).

    The reference appends all new tokens and then flushes the oldest ``G``
    while the window holds ``>= R`` tokens (cache/manager.py:226-243).
    """
    residual += new
    flushes = 0
    while residual >= R:
        residual -= G
        quantized += G
        flushes += 1
    return flushes, quantized, residual


class OracleCache:
    """One layer of the reference cache, restated on CPU tensors.

    Keeps what the reference discards (packed codes, scales, zeros per flush)
    next to what it serves (round-tripped fp32 history || fp32 residual), so
    both the state machine and the packed store of the CUDA cache can be
    checked.  Flush transform: keys chunk [B,H,G,D] -> transpose to [B,H,D,G]
    -> per-channel groups; values chunk [B,H,G,D] -> per-token groups of G
    channels (cache/manager.py:332-345).
    """

    def __init__(self, head_dim: int, group_size: int = 32,
                 residual_length: int = 128, rounding: str = "half_even"):
        assert head_dim % group_size == 0                      # manager.py:82
        assert group_size >= 4 and group_size % 4 == 0         # manager.py:84
        assert group_size <= residual_length                   # manager.py:86
        self.D, self.G, self.R = head_dim, group_size, residual_length
        self.rounding = rounding
        self.res_k: Optional[torch.Tensor] = None
        self.res_v: Optional[torch.Tensor] = None
        self.hist_k: List[torch.Tensor] = []   # round-tripped [B,H,G,D] chunks
        self.hist_v: List[torch.Tensor] = []
        self.k_packed: List[torch.Tensor] = []  # per flush [B,H,D,G/4]
        self.k_scales: List[torch.Tensor] = []  # per flush [B,H,D]
        self.k_zeros: List[torch.Tensor] = []
        self.v_packed: List[torch.Tensor] = []  # per flush [B,H,G,D/4]
        self.v_scales: List[torch.Tensor] = []  # per flush [B,H,G,D/G]
        self.v_zeros: List[torch.Tensor] = []
        self.flushes = 0

    @property
    def quantized_len(self) -> int:
        return self.flushes * self.G

    @property
    def residual_len(self) -> int:
        return 0 if self.res_k is None else self.res_k.shape[2]

    def append(self, new_k: torch.Tensor, new_v: torch.Tensor) -> None:
        new_k, new_v = new_k.float(), new_v.float()            # manager.py:210-214
        if self.res_k is None:
            self.res_k, self.res_v = new_k, new_v
        else:
            self.res_k = torch.cat([self.res_k, new_k], dim=2)  # manager.py:230
            self.res_v = torch.cat([self.res_v, new_v], dim=2)
        while self.res_k.shape[2] >= self.R:                   # manager.py:242
            self._flush()

    def _flush(self) -> None:
        G = self.G
        kc = self.res_k[:, :, :G, :].transpose(2, 3).contiguous()  # manager.py:332-334
        vc = self.res_v[:, :, :G, :].contiguous()                  # manager.py:341
        B, H, D, _ = kc.shape
        rk = quantize_groups(kc, G, self.rounding)
        rv = quantize_groups(vc, G, self.rounding)
        self.k_packed.append(rk["packed"].reshape(B, H, D, G // 4))
        self.k_scales.append(rk["scales"].reshape(B, H, D))
        self.k_zeros.append(rk["zeros"].reshape(B, H, D))
        self.v_packed.append(rv["packed"].reshape(B, H, G, D // 4))
        self.v_scales.append(rv["scales"].reshape(B, H, G, D // G))
        self.v_zeros.append(rv["zeros"].reshape(B, H, G, D // G))
        self.hist_k.append(roundtrip_groups(kc, G, self.rounding).transpose(2, 3))
        self.hist_v.append(roundtrip_groups(vc, G, self.rounding))
        self.res_k = self.res_k[:, :, G:, :].contiguous()          # manager.py:359
        self.res_v = self.res_v[:, :, G:, :].contiguous()
        self.flushes += 1

    def served(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """``history || residual`` as fp32 [B,H,T,D] (manager.py:263-286)."""
        pk = list(self.hist_k) + ([self.res_k] if self.residual_len else [])
        pv = list(self.hist_v) + ([self.res_v] if self.residual_len else [])
        return torch.cat(pk, dim=2), torch.cat(pv, dim=2)

    def stats_bytes(self) -> int:
        """Analytic packed-store bytes, manager.py:350-356."""
        if self.res_k is None:
            return 0
        B, H = self.res_k.shape[:2]
        D, G = self.D, self.G
        per = B * H * (D * (G // 4) + D * 8 + G * (D // 4) + G * (D // G) * 8)
        return per * self.flushes


# --------------------------------------------------------------------------
# Decode attention
# --------------------------------------------------------------------------

def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              dtype=torch.float32) -> torch.Tensor:
    """``softmax(q K^T * D**-0.5, dim=-1) V``
    (tests/integration/test_attention_fix.py:40-43).

    q [B,Hq,Lq,D]; k, v [B,Hkv,T,D].  With Hq > Hkv each KV head serves
    Hq/Hkv consecutive query heads (the grouped-query convention of the
    third-party model code the reference hands its cache to).  Evaluated as a
    grouped matmul, never materialising repeated K/V.
    """
    B, Hq, Lq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    qg = q.to(dtype).reshape(B, Hkv, rep * Lq, D)
    w = torch.matmul(qg, k.to(dtype).transpose(-2, -1)) * (D ** -0.5)
    w = torch.softmax(w, dim=-1)
    o = torch.matmul(w, v.to(dtype))
    return o.reshape(B, Hq, Lq, D)


def kivi_decode_attention(q: torch.Tensor, k_all: torch.Tensor, v_all: torch.Tensor,
                          n_quant: int, group_size: int,
                          rounding: str = "half_even", dtype=torch.float32
                          ) -> torch.Tensor:
    """Reference composition for one decode step over a KIVI cache.

    ``k_all``/``v_all`` [B,Hkv,T,D] hold the raw tokens; the first ``n_quant``
    (a multiple of G) are served round-tripped chunk by chunk exactly as the
    flush does (manager.py:332-345), the rest at full precision
    (manager.py:263-286); attention as in test_attention_fix.py:40-43.
    q [B,Hq,D] -> out [B,Hq,D].
    """
    G = group_size
    assert n_quant % G == 0
    kf, vf = k_all.float(), v_all.float()
    B, H, T, D = kf.shape
    if n_quant:
        kq = kf[:, :, :n_quant].reshape(B, H, n_quant // G, G, D)
        # keys: groups of G tokens per channel -> put tokens last, then flat.
        kq = roundtrip_groups(kq.transpose(3, 4).contiguous(), G, rounding).transpose(3, 4)
        kq = kq.reshape(B, H, n_quant, D)
        vq = roundtrip_groups(vf[:, :, :n_quant].contiguous(), G, rounding)
        kf = torch.cat([kq, kf[:, :, n_quant:]], dim=2)
        vf = torch.cat([vq, vf[:, :, n_quant:]], dim=2)
    return attention(q.float().unsqueeze(2), kf, vf, dtype=dtype).squeeze(2)


# --------------------------------------------------------------------------
# Seeded synthetic inputs (stand-in for the reference's GPT-2 benchmark data)
# --------------------------------------------------------------------------

def make_keys(B, H, S, D, seed, dtype=torch.float32) -> torch.Tensor:
    """N(0,1) keys with 4 seeded outlier channels per head scaled x10."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, H, S, D, generator=g, dtype=torch.float32)
    for h in range(H):
        ch = torch.randperm(D, generator=g)[:4]
        k[:, h, :, ch] *= 10.0
    return k.to(dtype)


def make_values(B, H, S, D, seed, dtype=torch.float32) -> torch.Tensor:
    """N(0,1) values with ceil(2% of tokens) per (b,h) scaled x8."""
    g = torch.Generator().manual_seed(seed + 1_000_003)
    v = torch.randn(B, H, S, D, generator=g, dtype=torch.float32)
    n = max(1, math.ceil(0.02 * S))
    for b in range(B):
        for h in range(H):
            tok = torch.randperm(S, generator=g)[:n]
            v[b, h, tok, :] *= 8.0
    return v.to(dtype)


def make_queries(B, Hq, D, seed, dtype=torch.float32) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 2_000_003)
    return torch.randn(B, Hq, D, generator=g, dtype=torch.float32).to(dtype)


# --------------------------------------------------------------------------
# Algorithmic byte counts used for the roofline
# --------------------------------------------------------------------------

def algorithmic_bytes_quantize(n_elem: int, group_size: int, in_bytes: int) -> int:
    """read input once, write codes, write fp32 scale+zero per group."""
    return n_elem * in_bytes + n_elem // 4 + (n_elem // group_size) * 8


def algorithmic_bytes_attention(B, Hkv, Hq, D, G, n_quant, n_res, t_bytes) -> int:
    """packed codes + fp32 scale/zero for K and V of every quantized token,
    the full-precision residual window, q in and out."""
    per_tok = D // 2 + 16 * D // G
    return B * Hkv * (n_quant * per_tok + n_res * 2 * D * t_bytes) + 2 * B * Hq * D * t_bytes


# --------------------------------------------------------------------------
# Next-token choice (src/kivi_sycl/generation/sampling.py:10-25) with the
# counter-based draw of include/kivi_cuda.h: kivi_sample_tokens
# --------------------------------------------------------------------------

def philox4x32_first_word(seed: int, step: int, row: int) -> int:
    """First output word of Philox4x32-10 (Salmon et al. 2011) with key = the two
    halves of ``seed`` and counter = (step lo, step hi, row, 0)."""
    M = 0xFFFFFFFF
    c = [step & M, (step >> 32) & M, row & M, 0]
    k = [seed & M, (seed >> 32) & M]
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & M, (p0 >> 32) ^ c[3] ^ k[1], p0 & M]
        k = [(k[0] + 0x9E3779B9) & M, (k[1] + 0xBB67AE85) & M]
    return c[0]


def sample_tokens(logits: torch.Tensor, temperature: float, top_k: Optional[int], do_sample: bool,
                  seed: int = 0, step: int = 0) -> torch.Tensor:
    """The reference's sample_token with its multinomial draw replaced by the
    inverse CDF (index order) at u = (w + 0.5) / 2^32, w = philox word of
    (seed, step, row).  logits [B, V] -> int64 [B]."""
    x = logits.float()
    if not do_sample:
        return x.argmax(dim=-1)
    x = x / max(temperature, 1e-8)
    if top_k:
        kth = x.topk(top_k, dim=-1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    w = torch.exp((x - x.amax(dim=-1, keepdim=True)).double())
    cdf = w.cumsum(dim=-1)
    out = torch.empty(x.shape[0], dtype=torch.int64)
    for b in range(x.shape[0]):
        u = (philox4x32_first_word(seed, step, b) + 0.5) / 4294967296.0
        out[b] = int(torch.searchsorted(cdf[b], torch.tensor(u * float(cdf[b, -1]), dtype=torch.float64), right=True))
    return out.clamp_max(x.shape[1] - 1)
