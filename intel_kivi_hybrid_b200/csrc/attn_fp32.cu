// Fused decode attention over the packed KIVI cache: CUDA-core fp32 kernel.
//
//   out = softmax(q K^T * D^-0.5) V   over [quantized history || residual ring]
// (formula: tests/integration/test_attention_fix.py:40-43; the operand is what
// cache/manager.py:263-286 would serve, but nothing is ever dequantized to
// memory).  Every number is fp32: codes are unpacked in registers, turned into
// k = code*scale + zero, and fed to fp32 FMAs, so this kernel holds the 1e-5
// tolerance of fp32 activations and covers every supported shape.  The
// tensor-core kernel in attn_mma.cu is the fast path for the Llama shape.
//
// Work split: grid = (splits, units).  The quantized history of a unit is cut
// into `nq_splits` runs of whole token groups; the residual ring is one more
// split.  Inside a CTA each warp walks its own groups with a private running
// (max, sum, output); warps are merged through shared memory and the CTA writes
// one partial (max, sum, unnormalised output) per query head to the workspace.
// merge_splits_kernel folds the partials (the only scratch memory of the op).
//
// Per 32-token chunk a warp does: lane = token for the q.k scores (each lane
// walks the D channels of its token), a warp max, exp2, then lane = 4 channels
// for p.V (each lane walks the chunk's tokens).
#include "kivi_common.cuh"

namespace kivi {


namespace {

constexpr int kWarps = 4;

template <int NREP, int DB>
__global__ void __launch_bounds__(kWarps * 32)
attn_fp32_kernel(kivi_layer L, int64_t quant_len, int res_start, int res_len,
                 const void* __restrict__ q, int q_dtype, float scale_log2,
                 int nq_splits, int groups_per_split, int split_base, int n_splits,
                 float* __restrict__ part_o, float* __restrict__ part_ml) {
    const int D = L.head_dim, G = L.group_size, Q = G / 4, W = D < 64 ? D : 64, ng = D / G;
    const int u = blockIdx.y, split = blockIdx.x + split_base;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t max_groups = L.max_tokens / G;

    extern __shared__ __align__(16) float smem[];
    float* q_s = smem;                                   // [NREP][D]
    float* sz_s = q_s + NREP * D + warp * 2 * D;         // per warp: scales[D], zeros[D]
    float* p_s = q_s + NREP * D + kWarps * 2 * D + warp * 32 * NREP;   // per warp [32][NREP]
    float* red_s = q_s + NREP * D + kWarps * 2 * D + kWarps * 32 * NREP;  // [kWarps][NREP][2] + [NREP][DB*128]

    for (int i = threadIdx.x; i < NREP * D; i += blockDim.x)
        q_s[i] = load_as_float(q, q_dtype, (int64_t)u * NREP * D + i);
    __syncthreads();

    float m[NREP], l[NREP], o[NREP][DB][4];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
        for (int b = 0; b < DB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[h][b][i] = 0.0f;
    }

    // softmax update for one chunk of <= 32 tokens whose raw scores sit in acc[]
    auto absorb_scores = [&](float (&acc)[NREP], bool valid) {
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            float s = valid ? acc[h] * scale_log2 : -INFINITY;
            float mx = s;
#pragma unroll
            for (int o_ = 16; o_ > 0; o_ >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o_));
            const float m_new = fmaxf(m[h], mx);            // finite: every chunk has >= 1 token
            const float alpha = exp2f(m[h] - m_new);        // exp2(-inf) = 0 on the first chunk
            const float p = valid ? exp2f(s - m_new) : 0.0f;
            m[h] = m_new;
            l[h] = l[h] * alpha + p;
#pragma unroll
            for (int b = 0; b < DB; ++b)
#pragma unroll
                for (int i = 0; i < 4; ++i) o[h][b][i] *= alpha;
            p_s[lane * NREP + h] = p;
        }
        __syncwarp();
    };

    if (split < nq_splits) {
        const int64_t n_groups = quant_len / G;
        const int64_t g_begin = (int64_t)split * groups_per_split;
        int64_t g_end = g_begin + groups_per_split;
        if (g_end > n_groups) g_end = n_groups;
        for (int64_t g = g_begin + warp; g < g_end; g += kWarps) {
            const int64_t gb = (int64_t)u * max_groups + g;
            const uint8_t* kb = L.k_codes + gb * (D * Q);
            __syncwarp();
            for (int d = lane; d < D; d += 32) {
                sz_s[d] = __ldg(L.k_scales + gb * D + d);
                sz_s[D + d] = __ldg(L.k_zeros + gb * D + d);
            }
            __syncwarp();
            for (int c0 = 0; c0 < G; c0 += 32) {
                const int tt = c0 + lane;
                const bool valid = tt < G;
                float acc[NREP];
#pragma unroll
                for (int h = 0; h < NREP; ++h) acc[h] = 0.0f;
                if (valid) {
                    const int j = tt / 4, e = tt % 4;
                    for (int d0 = 0; d0 < D; d0 += 4) {
                        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(kb + kblock_offset(d0, j, Q, W)));
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float code = (float)((w >> (8 * i + 2 * e)) & 3u);
                            const float k = fmaf(code, sz_s[d0 + i], sz_s[D + d0 + i]);
#pragma unroll
                            for (int h = 0; h < NREP; ++h) acc[h] = fmaf(q_s[h * D + d0 + i], k, acc[h]);
                        }
                    }
                }
                absorb_scores(acc, valid);
                const int ntok = G - c0 < 32 ? G - c0 : 32;
                const int64_t t0 = g * G + c0;
                const uint8_t* vcu = L.v_codes + (int64_t)u * L.max_tokens * (D / 4);
                const float* vsu = L.v_scales + (int64_t)u * L.max_tokens * ng;
                const float* vzu = L.v_zeros + (int64_t)u * L.max_tokens * ng;
                for (int tk = 0; tk < ntok; ++tk) {
                    float p[NREP];
#pragma unroll
                    for (int h = 0; h < NREP; ++h) p[h] = p_s[tk * NREP + h];
#pragma unroll
                    for (int b = 0; b < DB; ++b) {
                        const int byte = lane + 32 * b;
                        if (byte < D / 4) {
                            const uint32_t vb = __ldg(vcu + vcode_offset(t0 + tk, byte, D, G));
                            const int gd = (4 * byte) / G;
                            const int64_t mi = vmeta_index(t0 + tk, gd, D, G);
                            const float s = __ldg(vsu + mi);
                            const float z = __ldg(vzu + mi);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float v = fmaf((float)((vb >> (2 * i)) & 3u), s, z);
#pragma unroll
                                for (int h = 0; h < NREP; ++h) o[h][b][i] = fmaf(p[h], v, o[h][b][i]);
                            }
                        }
                    }
                }
                __syncwarp();
            }
        }
    } else {
        // residual ring, full precision (cache/manager.py:275-278)
        const int R = L.residual_cap;
        for (int c0 = warp * 32; c0 < res_len; c0 += kWarps * 32) {
            const int r = c0 + lane;
            const bool valid = r < res_len;
            float acc[NREP];
#pragma unroll
            for (int h = 0; h < NREP; ++h) acc[h] = 0.0f;
            if (valid) {
                const int slot = (res_start + r) % R;
                const int64_t base = ((int64_t)u * R + slot) * D;
                for (int d = 0; d < D; ++d) {
                    const float k = load_as_float(L.k_res, L.res_dtype, base + d);
#pragma unroll
                    for (int h = 0; h < NREP; ++h) acc[h] = fmaf(q_s[h * D + d], k, acc[h]);
                }
            }
            absorb_scores(acc, valid);
            const int ntok = res_len - c0 < 32 ? res_len - c0 : 32;
            for (int tk = 0; tk < ntok; ++tk) {
                const int slot = (res_start + c0 + tk) % R;
                const int64_t base = ((int64_t)u * R + slot) * D;
                float p[NREP];
#pragma unroll
                for (int h = 0; h < NREP; ++h) p[h] = p_s[tk * NREP + h];
#pragma unroll
                for (int b = 0; b < DB; ++b) {
                    const int byte = lane + 32 * b;
                    if (byte < D / 4) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float v = load_as_float(L.v_res, L.res_dtype, base + 4 * byte + i);
#pragma unroll
                            for (int h = 0; h < NREP; ++h) o[h][b][i] = fmaf(p[h], v, o[h][b][i]);
                        }
                    }
                }
            }
            __syncwarp();
        }
    }

    // ---- merge the warps of this CTA -------------------------------------
    float* ml_s = red_s;                         // [kWarps][NREP][2]
    float* o_s = red_s + kWarps * NREP * 2;      // [NREP][DB*128]
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        float ls = l[h];
#pragma unroll
        for (int o_ = 16; o_ > 0; o_ >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o_);
        if (lane == 0) { ml_s[(warp * NREP + h) * 2] = m[h]; ml_s[(warp * NREP + h) * 2 + 1] = ls; }
    }
    for (int i = threadIdx.x; i < NREP * DB * 128; i += blockDim.x) o_s[i] = 0.0f;
    __syncthreads();
    float M[NREP];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        float mm = -INFINITY;
        for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, ml_s[(w * NREP + h) * 2]);
        M[h] = mm;
    }
    for (int w = 0; w < kWarps; ++w) {
        if (warp == w) {
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                const float f = (m[h] == -INFINITY) ? 0.0f : exp2f(m[h] - M[h]);
#pragma unroll
                for (int b = 0; b < DB; ++b)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        o_s[h * DB * 128 + (lane + 32 * b) * 4 + i] += o[h][b][i] * f;
            }
        }
        __syncthreads();
    }
    const int64_t pbase = ((int64_t)u * n_splits + split) * NREP;
    for (int i = threadIdx.x; i < NREP * D; i += blockDim.x) {
        const int h = i / D, d = i % D;
        part_o[(pbase + h) * D + d] = o_s[h * DB * 128 + d];
    }
    if (threadIdx.x < NREP) {
        const int h = threadIdx.x;
        float ls = 0.0f;
        for (int w = 0; w < kWarps; ++w) {
            const float mw = ml_s[(w * NREP + h) * 2];
            if (mw != -INFINITY) ls += ml_s[(w * NREP + h) * 2 + 1] * exp2f(mw - M[h]);
        }
        part_ml[(pbase + h) * 2] = M[h];
        part_ml[(pbase + h) * 2 + 1] = ls;
    }
}

}  // namespace

namespace {

__device__ __forceinline__ void store_quad(void* p, int dtype, int64_t i, float4 v);

// out[u][h][:] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
// One warp per output row (row = u*n_rep + h), kMergeWarps rows per CTA; partials
// laid out [(u*n_splits + s)*n_rep + h].  Lane s holds (m_s, l_s) and the weight
// of split s, the maximum and the denominator are warp reductions, and every
// lane folds four channels with 16-byte loads, the weights handed round by
// shuffle.  `sink(index, float4)` receives the four output elements starting at
// index = row*D + d (d a multiple of four; head_dim is a multiple of four).
constexpr int kMergeWarps = 8;

template <typename Sink>
__device__ __forceinline__ void merge_row(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          int n_splits, int nrep, int64_t row, int D, const Sink& sink,
                                          float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t u = row / nrep;
    const int h = (int)(row - u * nrep);
    const int64_t row0 = u * n_splits * nrep + h;            // + s*nrep
    float M = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, part_ml[(row0 + (int64_t)s * nrep) * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    for (int d0 = 0; d0 < D; d0 += 128) {
        const int d = d0 + 4 * lane;
        const bool active = d < D;
        float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
        float den = 0.0f;
        for (int s0 = 0; s0 < n_splits; s0 += 32) {
            const int s = s0 + lane;
            float wgt = 0.0f;
            if (s < n_splits) {
                const float2 ml = *reinterpret_cast<const float2*>(part_ml + (row0 + (int64_t)s * nrep) * 2);
                wgt = (ml.x == -INFINITY) ? 0.0f : exp2f(ml.x - M);
                den = fmaf(wgt, ml.y, den);
            }
            const int cnt = min(32, n_splits - s0);
            const float* src = part_o + (row0 + (int64_t)s0 * nrep) * D + (active ? d : 0);
            // eight partial rows in flight per lane (a unit cut into a hundred pieces
            // would otherwise pay a hundred load latencies in a row); rows past the
            // end are the last row again, with weight zero
            for (int i = 0; i < cnt; i += 8) {
                float4 v[8];
                float w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int k = i + j < cnt ? i + j : cnt - 1;
                    v[j] = *reinterpret_cast<const float4*>(src + (int64_t)k * nrep * D);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float wj = __shfl_sync(0xffffffffu, wgt, (i + j) & 31);
                    w[j] = i + j < cnt ? wj : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    a0.x = fmaf(v[j].x, w[j], a0.x); a0.y = fmaf(v[j].y, w[j], a0.y);
                    a0.z = fmaf(v[j].z, w[j], a0.z); a0.w = fmaf(v[j].w, w[j], a0.w);
                    a1.x = fmaf(v[j + 1].x, w[j + 1], a1.x); a1.y = fmaf(v[j + 1].y, w[j + 1], a1.y);
                    a1.z = fmaf(v[j + 1].z, w[j + 1], a1.z); a1.w = fmaf(v[j + 1].w, w[j + 1], a1.w);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        const float inv = 1.0f / den;
        // natural-log sum of exponentials of the scaled scores (M and den live in the log2 domain)
        if (lse != nullptr && lane == 0 && d0 == 0) lse[row] = (M + log2f(den)) * 0.6931471805599453f;
        if (active)
            sink(row * D + d, make_float4((a0.x + a1.x) * inv, (a0.y + a1.y) * inv, (a0.z + a1.z) * inv, (a0.w + a1.w) * inv));
    }
}

// The same fold with all kMergeWarps warps of a CTA on ONE row, for rows with
// many partials (few units cut into many pieces): warp w folds pieces w, w + 8,
// ... with eight loads in flight, the warps' sums meet in shared memory and are
// added in warp order.  (A different summation order than merge_row: which of
// the two a call uses depends on its piece count alone.)
constexpr int kMergeWideFrom = 17;            // partials per row from which the CTA-wide fold is used

template <typename Sink>
__device__ __forceinline__ void merge_row_wide(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                               int n_splits, int nrep, int64_t row, int D, const Sink& sink,
                                               float* __restrict__ lse, float (*fold_s)[128]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t u = row / nrep;
    const int h = (int)(row - u * nrep);
    const int64_t row0 = u * n_splits * nrep + h;            // + s*nrep
    // every warp works out the maximum and the denominator itself (same loads, same order, same bits)
    float M = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, part_ml[(row0 + (int64_t)s * nrep) * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float den = 0.0f;
    for (int s = lane; s < n_splits; s += 32) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (row0 + (int64_t)s * nrep) * 2);
        den = fmaf((ml.x == -INFINITY) ? 0.0f : exp2f(ml.x - M), ml.y, den);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    const float inv = 1.0f / den;
    const int n_mine = warp < n_splits ? (n_splits - warp + kMergeWarps - 1) / kMergeWarps : 0;
    for (int d0 = 0; d0 < D; d0 += 128) {
        const int d = d0 + 4 * lane;
        const bool active = d < D;
        float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
        const float* src = part_o + row0 * D + (active ? d : 0);
        for (int i = 0; i < n_mine; i += 8) {
            float4 v[8];
            float w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int s = warp + kMergeWarps * (i + j < n_mine ? i + j : n_mine - 1);
                v[j] = *reinterpret_cast<const float4*>(src + (int64_t)s * nrep * D);
                const float ms = part_ml[(row0 + (int64_t)s * nrep) * 2];
                w[j] = (i + j < n_mine && ms != -INFINITY) ? exp2f(ms - M) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                a0.x = fmaf(v[j].x, w[j], a0.x); a0.y = fmaf(v[j].y, w[j], a0.y);
                a0.z = fmaf(v[j].z, w[j], a0.z); a0.w = fmaf(v[j].w, w[j], a0.w);
                a1.x = fmaf(v[j + 1].x, w[j + 1], a1.x); a1.y = fmaf(v[j + 1].y, w[j + 1], a1.y);
                a1.z = fmaf(v[j + 1].z, w[j + 1], a1.z); a1.w = fmaf(v[j + 1].w, w[j + 1], a1.w);
            }
        }
        *reinterpret_cast<float4*>(&fold_s[warp][4 * lane]) = make_float4(a0.x + a1.x, a0.y + a1.y, a0.z + a1.z, a0.w + a1.w);
        __syncthreads();
        if (warp == 0) {
            float4 t = *reinterpret_cast<const float4*>(&fold_s[0][4 * lane]);
#pragma unroll
            for (int w2 = 1; w2 < kMergeWarps; ++w2) {
                const float4 b = *reinterpret_cast<const float4*>(&fold_s[w2][4 * lane]);
                t.x += b.x; t.y += b.y; t.z += b.z; t.w += b.w;
            }
            // natural-log sum of exponentials of the scaled scores (M and den live in the log2 domain)
            if (lse != nullptr && lane == 0 && d0 == 0) lse[row] = (M + log2f(den)) * 0.6931471805599453f;
            if (active) sink(row * D + d, make_float4(t.x * inv, t.y * inv, t.z * inv, t.w * inv));
        }
        __syncthreads();                                  // fold_s is rewritten by the next 128 channels
    }
}

// four consecutive output elements starting at element i (i % 4 == 0): one 8- or
// 16-byte store when the buffer allows it
__device__ __forceinline__ void store_quad(void* p, int dtype, int64_t i, float4 v) {
    if (dtype == KIVI_BF16) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p) + i;
        if ((reinterpret_cast<uintptr_t>(o) & 7u) == 0) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 w;
            w.x = *reinterpret_cast<const uint32_t*>(&lo); w.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(o) = w;
        } else {
            o[0] = __float2bfloat16_rn(v.x); o[1] = __float2bfloat16_rn(v.y);
            o[2] = __float2bfloat16_rn(v.z); o[3] = __float2bfloat16_rn(v.w);
        }
    } else {
        float* o = reinterpret_cast<float*>(p) + i;
        if ((reinterpret_cast<uintptr_t>(o) & 15u) == 0) *reinterpret_cast<float4*>(o) = v;
        else { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
    }
}

struct LocalSink {
    void* out;
    int out_dtype;
    __device__ void operator()(int64_t i, float4 v) const { store_quad(out, out_dtype, i, v); }
};

__global__ void __launch_bounds__(kMergeWarps * 32)
merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    void* __restrict__ out, int out_dtype, int n_splits, int nrep, int64_t rows, int D,
                    float* __restrict__ lse) {
    // launched with programmatic stream serialization: the launch may overlap the
    // tail of the attention kernel, the partials may not be read before that
    // kernel has completed
    __shared__ __align__(16) float fold_s[kMergeWarps][128];
    cudaGridDependencySynchronize();
    if (n_splits >= kMergeWideFrom) {                     // grid = rows: the whole CTA on one row
        merge_row_wide(part_o, part_ml, n_splits, nrep, (int64_t)blockIdx.x, D, LocalSink{out, out_dtype}, lse, fold_s);
        return;
    }
    const int64_t row = (int64_t)blockIdx.x * kMergeWarps + (threadIdx.x >> 5);
    if (row < rows) merge_row(part_o, part_ml, n_splits, nrep, row, D, LocalSink{out, out_dtype}, lse);
}

// ---- merge + all-gather over peer memory -------------------------------------------
// The same fold, but every output row is stored into the gathered buffer of
// every rank (plain stores through peer-mapped pointers).  When the last CTA of
// the grid has finished, lane r of its first warp publishes this rank's epoch in
// rank r's flag array and, if asked, waits (bounded) until rank r has published
// it here: one fence, then all flags and all waits side by side.
__device__ unsigned g_gather_done = 0;      // CTAs of the running launch that have stored their row
__device__ int g_gather_fault = 0;

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct PeerSink {
    kivi_peer_gather g;
    int out_dtype;
    int64_t base;              // element offset of this rank's first row in a gathered buffer
    int64_t alt;               // byte offset of the buffer this call writes (device-kept epoch: odd calls)
    __device__ void operator()(int64_t i, float4 v) const {
#pragma unroll
        for (int r = 0; r < KIVI_PEER_MAX_WORLD; ++r)
            if (r < g.world) store_quad(reinterpret_cast<uint8_t*>(g.out_ptrs[r]) + alt, out_dtype, base + i, v);
    }
};

constexpr uint32_t kPeerSpinLimit = 5u << 20;      // default bound: x 200 ns sleeps, about a second

__global__ void __launch_bounds__(kMergeWarps * 32)
merge_gather_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    kivi_peer_gather g, int out_dtype, int n_splits, int nrep, int64_t rows, int D) {
    cudaGridDependencySynchronize();
    // Epoch kept on the device (a call replayed from a CUDA graph): every CTA
    // reads the counter here; the last CTA stores it back after all CTAs have
    // counted themselves in, that is after all of them have read it.
    uint32_t epoch = g.epoch;
    int64_t alt = 0;
    if (g.epoch_dev != nullptr) {
        epoch = *reinterpret_cast<const volatile uint32_t*>(g.epoch_dev) + 1u;
        alt = (epoch & 1u) ? g.alt_bytes : 0;
    }
    __shared__ __align__(16) float fold_s[kMergeWarps][128];
    const PeerSink sink{g, out_dtype, g.unit_offset * (int64_t)nrep * D, alt};
    if (n_splits >= kMergeWideFrom) {                     // grid = rows: the whole CTA on one row
        merge_row_wide(part_o, part_ml, n_splits, nrep, (int64_t)blockIdx.x, D, sink, nullptr, fold_s);
    } else {
        const int64_t row = (int64_t)blockIdx.x * kMergeWarps + (threadIdx.x >> 5);
        if (row < rows) merge_row(part_o, part_ml, n_splits, nrep, row, D, sink, nullptr);
    }
    __syncthreads();                                  // the CTA's stores are issued
    if (threadIdx.x >= 32) return;                    // warp 0 carries the protocol
    const int lane = threadIdx.x;
    const unsigned total = gridDim.x;
    unsigned last = 0;
    if (lane == 0) {
        __threadfence_system();                       // ... and ordered before the count below, system-wide
        last = atomicAdd(&g_gather_done, 1u) + 1u == total;
        if (last) {
            g_gather_done = 0;                        // re-armed for the next launch (stream order)
            if (g.epoch_dev != nullptr) *g.epoch_dev = epoch;
            __threadfence_system();                   // what the other CTAs published comes before the flags
        }
    }
    __syncwarp();
    if (!__shfl_sync(0xffffffffu, last, 0)) return;
    // lane r tells rank r and then waits for rank r: the flags travel, and are polled, side by side
    const bool has_peer = lane < g.world;
    if (has_peer) st_relaxed_sys(g.flag_ptrs[lane] + g.rank, epoch);
    if (!g.wait) return;
    const uint32_t limit = g.spin_limit ? g.spin_limit : kPeerSpinLimit;
    uint64_t t0 = 0;
    if (g.wait_stats && lane == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    if (has_peer) {
        const uint32_t* mine = g.flag_ptrs[g.rank] + lane;
        uint32_t it = 0;
        while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++it > limit) { atomicOr(&g_gather_fault, 2); break; }
            __nanosleep(200);
        }
    }
    __syncwarp();
    if (g.wait_stats && lane == 0) {
        uint64_t t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        g.wait_stats[0] += t1 - t0;        // one thread of one CTA per launch, launches are stream-ordered
        g.wait_stats[1] += 1;
    }
}

}  // namespace

int gather_fault_word(int* out) {
    KIVI_CUDA_OK(cudaMemcpyFromSymbol(out, g_gather_fault, sizeof(int)));
    return KIVI_OK;
}

int gather_fault_clear() {
    const int zero = 0;
    KIVI_CUDA_OK(cudaMemcpyToSymbol(g_gather_fault, &zero, sizeof(int)));
    return KIVI_OK;
}

// merge of the split partials into `out`, or (gather != nullptr) into every
// rank's gathered buffer; queued behind the attention kernel with programmatic
// stream serialization, so its launch latency overlaps that kernel's tail
int run_merge(const float* part_o, const float* part_ml, void* out, const kivi_peer_gather* gather, float* lse,
              int out_dtype, int num_units, int n_rep, int n_splits, int D, cudaStream_t st) {
    const int64_t rows = (int64_t)num_units * n_rep;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_splits >= kMergeWideFrom ? rows : (rows + kMergeWarps - 1) / kMergeWarps));
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (gather) {
        kivi_peer_gather g = *gather;
        KIVI_CUDA_OK(cudaLaunchKernelEx(&cfg, merge_gather_kernel, part_o, part_ml, g, out_dtype, n_splits, n_rep, rows, D));
    } else {
        KIVI_CUDA_OK(cudaLaunchKernelEx(&cfg, merge_splits_kernel, part_o, part_ml, out, out_dtype, n_splits, n_rep, rows, D, lse));
    }
    return KIVI_OK;
}

// ---- token shards: combine attention computed over disjoint token ranges -----------
// parts [n_shards][rows][D + 1] fp32: D outputs then the natural-log sum of
// exponentials of the shard (-inf for a shard that attended to nothing).
// out[row] = sum_i out_i * exp(lse_i - LSE) / sum_i exp(lse_i - LSE); one warp per row.
__global__ void __launch_bounds__(128)
merge_token_shards_kernel(const float* __restrict__ parts, int n_shards, int64_t rows, int D,
                          void* __restrict__ out, int out_dtype, float* __restrict__ lse_out) {
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int64_t stride = rows * (D + 1);
    float M = -INFINITY;
    for (int i = 0; i < n_shards; ++i) M = fmaxf(M, parts[i * stride + row * (D + 1) + D]);
    float den = 0.0f;
    for (int i = 0; i < n_shards; ++i) {
        const float l = parts[i * stride + row * (D + 1) + D];
        den += (l == -INFINITY) ? 0.0f : expf(l - M);
    }
    for (int d = lane; d < D; d += 32) {
        float acc = 0.0f;
        for (int i = 0; i < n_shards; ++i) {
            const float l = parts[i * stride + row * (D + 1) + D];
            if (l != -INFINITY) acc = fmaf(parts[i * stride + row * (D + 1) + d], expf(l - M), acc);
        }
        store_from_float(out, out_dtype, row * D + d, acc / den);
    }
    if (lse_out != nullptr && lane == 0) lse_out[row] = M + logf(den);
}

int run_merge_token_shards(const float* parts, int n_shards, int64_t rows, int D, void* out, int out_dtype,
                           float* lse_out, cudaStream_t st) {
    merge_token_shards_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(parts, n_shards, rows, D, out, out_dtype, lse_out);
    KIVI_LAUNCH_OK();
    return KIVI_OK;
}

template <int NREP>
static int launch_fp32(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                       const void* q, int q_dtype, float scale_log2, int nq_splits, int gps,
                       int n_splits, float* part_o, float* part_ml, cudaStream_t st,
                       int split_base = 0, int grid_x = -1) {
    const int D = L->head_dim;
    const int DB = D > 128 ? 2 : 1;
    const size_t smem = sizeof(float) * ((size_t)NREP * D + kWarps * 2 * D + kWarps * 32 * NREP +
                                         kWarps * NREP * 2 + (size_t)NREP * DB * 128);
    dim3 grid((unsigned)(grid_x < 0 ? n_splits : grid_x), (unsigned)L->num_units);
    if (DB == 1) {
        if (smem > 48 * 1024) KIVI_CUDA_OK(cudaFuncSetAttribute(attn_fp32_kernel<NREP, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attn_fp32_kernel<NREP, 1><<<grid, kWarps * 32, smem, st>>>(*L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, split_base, n_splits, part_o, part_ml);
    } else {
        if (smem > 48 * 1024) KIVI_CUDA_OK(cudaFuncSetAttribute(attn_fp32_kernel<NREP, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attn_fp32_kernel<NREP, 2><<<grid, kWarps * 32, smem, st>>>(*L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, split_base, n_splits, part_o, part_ml);
    }
    KIVI_LAUNCH_OK();
    return KIVI_OK;
}

int run_attn_fp32(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                  const void* q, int q_dtype, int n_rep, float scale_log2, int nq_splits, int gps,
                  int n_splits, float* part_o, float* part_ml, cudaStream_t st) {
    switch (n_rep) {
        case 1: return launch_fp32<1>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 2: return launch_fp32<2>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 3: return launch_fp32<3>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 4: return launch_fp32<4>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 5: return launch_fp32<5>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 6: return launch_fp32<6>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 7: return launch_fp32<7>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        case 8: return launch_fp32<8>(L, quant_len, res_start, res_len, q, q_dtype, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
        default: break;
    }
    set_error("n_rep (%d) outside 1..8", n_rep);
    return KIVI_ERR_UNSUPPORTED;
}

}  // namespace kivi
