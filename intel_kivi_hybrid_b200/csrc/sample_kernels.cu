// Next-token choice on the device: argmax, or temperature / top-k / multinomial
// sampling over [batch, vocab] logits, one CTA per batch row.
//
// Same arithmetic as the reference's sample_token
// (src/kivi_sycl/generation/sampling.py:10-25): logits / max(temperature, 1e-8),
// everything below the k-th largest scaled logit masked out (ties with the k-th
// are kept, as `logits < kth` does), softmax, one draw.  The draw is the inverse
// CDF in index order of a counter-based uniform number (Philox4x32-10 keyed by
// (seed), counter (step, row)), so a CPU restatement reproduces it without
// sharing any generator state, and the ids never have to leave the device.
#include "kivi_common.cuh"

namespace kivi {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float logit_at(const void* p, int dtype, int64_t i) { return load_as_float(p, dtype, i); }

// order-preserving map float -> uint32 (larger float, larger key); NaN sorts above +inf
__device__ __forceinline__ uint32_t ordered_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) { return __umulhi(a, b); }

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"):
// returns the first of the four output words
__device__ uint32_t philox_first_word(uint64_t seed, uint64_t step, uint32_t row) {
    uint32_t c0 = (uint32_t)step, c1 = (uint32_t)(step >> 32), c2 = row, c3 = 0u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = mulhi32(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = mulhi32(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c0;
}

struct MaxIdx { float v; int i; };
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {      // larger value, then smaller index; NaN never wins
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const void* __restrict__ logits, int dtype, int vocab, int64_t row_stride,
              float temperature, int top_k, int do_sample, uint64_t seed, uint64_t step, int64_t* __restrict__ ids) {
    __shared__ unsigned hist[256];
    __shared__ float red_f[kThreads / 32];
    __shared__ int red_i[kThreads / 32];
    __shared__ double scan_s[kThreads];
    __shared__ double tgt[2];                               // (target mass, total mass)
    __shared__ uint32_t sel_prefix;
    __shared__ int sel_remaining, pick_s;
    // the reference divides: logits / max(temperature, 1e-8)
    auto scaled = [&](int i) { return __fdiv_rn(logit_at(logits, dtype, (int64_t)blockIdx.x * row_stride + i), temperature); };
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t base = (int64_t)row * row_stride;

    // ---- row maximum and its first index (also the argmax answer) ----------------
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += kThreads) best = better(best, MaxIdx{logit_at(logits, dtype, base + i), i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        best = better(best, MaxIdx{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    if (lane == 0) { red_f[warp] = best.v; red_i[warp] = best.i; }
    __syncthreads();
    best = MaxIdx{red_f[0], red_i[0]};
    for (int w = 1; w < kThreads / 32; ++w) best = better(best, MaxIdx{red_f[w], red_i[w]});
    if (best.i == 0x7fffffff) best.i = 0;                  // a row of NaNs / -inf
    if (!do_sample) {
        if (tid == 0) ids[row] = best.i;
        return;
    }

    // ---- k-th largest scaled logit: radix select on the ordered keys, 8 bits a pass --
    float kth = -INFINITY;
    if (top_k > 0 && top_k < vocab) {
        if (tid == 0) { sel_prefix = 0u; sel_remaining = top_k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int b = tid; b < 256; b += kThreads) hist[b] = 0u;
            __syncthreads();
            const uint32_t prefix = sel_prefix;
            const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < vocab; i += kThreads) {
                const uint32_t key = ordered_key(scaled(i));
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                int need = sel_remaining, b = 255;
                for (; b > 0; --b) {
                    if ((int)hist[b] >= need) break;
                    need -= (int)hist[b];
                }
                sel_prefix = prefix | ((uint32_t)b << shift);
                sel_remaining = need;
            }
            __syncthreads();
        }
        kth = key_to_float(sel_prefix);
    }

    // ---- softmax weights over the kept entries, contiguous chunk per thread -------
    const float m = __fdiv_rn(best.v, temperature);
    const int chunk = (vocab + kThreads - 1) / kThreads;
    const int i0 = tid * chunk, i1 = min(vocab, i0 + chunk);
    double mine = 0.0;
    for (int i = i0; i < i1; ++i) {
        const float x = scaled(i);
        if (x >= kth) mine += (double)expf(x - m);
    }
    scan_s[tid] = mine;
    if (tid == 0) pick_s = -1;
    __syncthreads();
    if (tid == 0) {                                         // 256 numbers: a serial scan keeps the order fixed
        double run = 0.0;
        for (int t = 0; t < kThreads; ++t) { const double v = scan_s[t]; scan_s[t] = run; run += v; }
        const uint32_t r = philox_first_word(seed, step, (uint32_t)row);
        tgt[0] = ((double)r + 0.5) * (1.0 / 4294967296.0) * run;
        tgt[1] = run;
    }
    __syncthreads();
    const double target = tgt[0], before = scan_s[tid];
    // exactly one chunk has before <= target < before + mine (masses are >= 0 and
    // target < total); it walks its kept entries until the running mass passes the target
    if (mine > 0.0 && before <= target && target < before + mine) {
        double run = before;
        int pick = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            const float x = scaled(i);
            if (x >= kth) {
                last_kept = i;
                run += (double)expf(x - m);
                if (run > target) { pick = i; break; }
            }
        }
        pick_s = pick >= 0 ? pick : last_kept;              // (the walk re-adds the same numbers: pick is found)
    }
    __syncthreads();
    // no chunk claimed the target (total mass 0 or not finite): fall back to the argmax
    if (tid == 0) ids[row] = pick_s >= 0 ? pick_s : best.i;
}

}  // namespace

int run_sample(const void* logits, int dtype, int batch, int vocab, int64_t row_stride, float temperature, int top_k,
               int do_sample, uint64_t seed, uint64_t step, int64_t* ids, cudaStream_t st) {
    const float t = temperature > 1e-8f ? temperature : 1e-8f;
    sample_kernel<<<batch, kThreads, 0, st>>>(logits, dtype, vocab, row_stride, t, top_k, do_sample, seed, step, ids);
    KIVI_LAUNCH_OK();
    return KIVI_OK;
}

}  // namespace kivi
