// Device-resident KIVI cache of one layer: on-device flush of whole token
// groups into the packed store, ring append, compatibility materialisation.
//
// Replaces the storage side of the reference's KiviCache
// (src/kivi_sycl/cache/manager.py:162-249 add_tokens, :309-374 _flush_group):
// there the residual lives on the CPU and each flush is an H2D copy, a blocking
// kernel, a D2H copy and an O(T) concatenation; here the host only does the
// counter arithmetic and enqueues kernels.
//
// A flush reads its tokens from the "virtual sequence" [live ring tokens in age
// order, then the new tokens], so one launch covers both a single decode flush
// (all G tokens in the ring) and a bulk prefill (thousands of groups cut
// straight out of the model's [units, S, D] tensor, the rest appended).
#include "kivi_common.cuh"

#ifndef KIVI_STAGE_F32
#define KIVI_STAGE_F32 true
#endif
#ifndef KIVI_STAGE_BF16
#define KIVI_STAGE_BF16 false
#endif

namespace kivi {
namespace {

struct TokenSource {
    const void* ring;     // [units][R][D] of ring_dtype
    const void* fresh;    // new tokens
    int ring_dtype, fresh_dtype;
    int R, D;
    int res_start, res_len;
    int64_t unit_stride, tok_stride;   // of `fresh`, in elements
};

// element d of virtual token tau of unit u
__device__ __forceinline__ float src_load(const TokenSource& s, int u, int64_t tau, int d) {
    if (tau < s.res_len) {
        int slot = (int)((s.res_start + tau) % s.R);
        return load_as_float(s.ring, s.ring_dtype, ((int64_t)u * s.R + slot) * s.D + d);
    }
    return load_as_float(s.fresh, s.fresh_dtype, (int64_t)u * s.unit_stride + (tau - s.res_len) * s.tok_stride + d);
}

template <typename T> struct Load8;
template <> struct Load8<float> {
    __device__ static void run(const float* p, float (&v)[8]) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct Load8<__nv_bfloat16> {
    __device__ static void run(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
};

// Keys of one token group of one unit: thread d owns channel d, reads the G
// tokens of its channel (a warp reads 32 consecutive channels of one token per
// instruction), quantizes them over the token axis, and the CTA writes one key
// block.  Grid: (groups, units).  GT > 0 keeps the group in registers.
template <int GT, bool HALF_EVEN>
__global__ void __launch_bounds__(256)
flush_keys_kernel(TokenSource src, uint8_t* __restrict__ k_codes, float* __restrict__ k_scales,
                  float* __restrict__ k_zeros, int64_t max_groups, int64_t group0, int G) {
    extern __shared__ __align__(16) uint8_t s_block[];   // D*G/4 bytes
    const int D = src.D;
    const int u = blockIdx.y;
    const int64_t g = group0 + blockIdx.x;                // destination group index
    const int64_t tau0 = (int64_t)blockIdx.x * G;         // first virtual token
    const int Q = G / 4, W = D < 64 ? D : 64;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float mn = 1e30f, mx = -1e30f;
        float x[GT > 0 ? GT : 1];
        if (GT > 0) {
#pragma unroll
            for (int t = 0; t < GT; ++t) x[t] = src_load(src, u, tau0 + t, d);
#pragma unroll
            for (int t = 0; t < GT; ++t) { mn = fminf(mn, x[t]); mx = fmaxf(mx, x[t]); }
        } else {
            for (int t = 0; t < G; ++t) {
                float v = src_load(src, u, tau0 + t, d);
                mn = fminf(mn, v); mx = fmaxf(mx, v);
            }
        }
        const float scale = group_scale(mn, mx);
        const float rcp = group_rcp(scale);
        k_scales[((int64_t)u * max_groups + g) * D + d] = scale;
        k_zeros[((int64_t)u * max_groups + g) * D + d] = mn;
        if (GT > 0) {
#pragma unroll
            for (int j = 0; j < GT / 4; ++j) {
                float q0 = code_magic<HALF_EVEN>(x[4 * j], mn, scale, rcp);
                float q1 = code_magic<HALF_EVEN>(x[4 * j + 1], mn, scale, rcp);
                float q2 = code_magic<HALF_EVEN>(x[4 * j + 2], mn, scale, rcp);
                float q3 = code_magic<HALF_EVEN>(x[4 * j + 3], mn, scale, rcp);
                s_block[kblock_offset(d, j, Q, W)] =
                    (uint8_t)pack4_magic(q0, q1, q2, q3);
            }
        } else {
            for (int j = 0; j < Q; ++j) {
                uint32_t byte = 0;
                for (int e = 0; e < 4; ++e) {
                    const float q = code_magic<HALF_EVEN>(src_load(src, u, tau0 + 4 * j + e, d), mn, scale, rcp);
                    byte |= (__float_as_uint(q) & 3u) << (2 * e);
                }
                s_block[kblock_offset(d, j, Q, W)] = (uint8_t)byte;
            }
        }
    }
    __syncthreads();
    const int block_bytes = D * Q;
    uint8_t* dst = k_codes + ((int64_t)u * max_groups + g) * block_bytes;
    if (block_bytes % 16 == 0) {
        for (int i = threadIdx.x * 16; i < block_bytes; i += blockDim.x * 16)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(s_block + i);
    } else {
        for (int i = threadIdx.x; i < block_bytes; i += blockDim.x) dst[i] = s_block[i];
    }
}

// Keys, fast path for D = 128, G = 32: the CTA stages the 32-token x 128-channel
// tile of its group in shared memory with 128-bit loads (a token row is
// contiguous in both sources), then thread d walks column d (conflict-free:
// a warp reads 32 consecutive elements of one row), quantizes it over the 32
// tokens and the CTA writes one key block with 128-bit stores.
template <typename TR, typename TF, bool HALF_EVEN>
__global__ void __launch_bounds__(128)
flush_keys_fast_kernel(TokenSource src, uint8_t* __restrict__ k_codes, float* __restrict__ k_scales,
                       float* __restrict__ k_zeros, int64_t max_groups, int64_t group0) {
    constexpr int D = 128, G = 32, Q = 8;
    __shared__ __align__(16) float s_tile[G][D + 4];     // +4: rows start 16 bytes apart in bank space
    __shared__ __align__(16) uint8_t s_block[D * Q];
    const int u = blockIdx.y;
    const int64_t g = group0 + blockIdx.x;
    const int64_t tau0 = (int64_t)blockIdx.x * G;
    // 32 rows x 16 pieces of 8 elements = 512 pieces, 4 per thread
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int piece = it * 128 + threadIdx.x;
        const int t = piece >> 4, c = (piece & 15) * 8;
        const int64_t tau = tau0 + t;
        float v[8];
        if (tau < src.res_len) {
            const int slot = (int)((src.res_start + tau) % src.R);
            Load8<TR>::run(reinterpret_cast<const TR*>(src.ring) + ((int64_t)u * src.R + slot) * D + c, v);
        } else {
            Load8<TF>::run(reinterpret_cast<const TF*>(src.fresh) + (int64_t)u * src.unit_stride +
                               (tau - src.res_len) * src.tok_stride + c, v);
        }
        *reinterpret_cast<float4*>(&s_tile[t][c]) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(&s_tile[t][c + 4]) = make_float4(v[4], v[5], v[6], v[7]);
    }
    __syncthreads();
    const int d = threadIdx.x;
    float x[G];
    float mn = 1e30f, mx = -1e30f;
#pragma unroll
    for (int t = 0; t < G; ++t) { x[t] = s_tile[t][d]; mn = fminf(mn, x[t]); mx = fmaxf(mx, x[t]); }
    const float scale = group_scale(mn, mx);
    const float rcp = group_rcp(scale);
    k_scales[((int64_t)u * max_groups + g) * D + d] = scale;
    k_zeros[((int64_t)u * max_groups + g) * D + d] = mn;
#pragma unroll
    for (int j = 0; j < Q; ++j) {
        const float q0 = code_magic<HALF_EVEN>(x[4 * j], mn, scale, rcp), q1 = code_magic<HALF_EVEN>(x[4 * j + 1], mn, scale, rcp);
        const float q2 = code_magic<HALF_EVEN>(x[4 * j + 2], mn, scale, rcp), q3 = code_magic<HALF_EVEN>(x[4 * j + 3], mn, scale, rcp);
        s_block[kblock_offset(d, j, Q, 64)] = (uint8_t)pack4_magic(q0, q1, q2, q3);
    }
    __syncthreads();
    uint8_t* dst = k_codes + ((int64_t)u * max_groups + g) * (D * Q);
    if (threadIdx.x < 64)
        *reinterpret_cast<uint4*>(dst + threadIdx.x * 16) = *reinterpret_cast<const uint4*>(s_block + threadIdx.x * 16);
}

// Values: one thread per (token, channel group); groups of G consecutive
// channels of one token (quantize_kernels.cpp:88-103).  Lanes of a warp take
// consecutive channel groups, so a warp covers 32*G consecutive elements.
template <bool HALF_EVEN>
__global__ void __launch_bounds__(256)
flush_values_kernel(TokenSource src, uint8_t* __restrict__ v_codes, float* __restrict__ v_scales,
                    float* __restrict__ v_zeros, int64_t max_tokens, int64_t tok0,
                    int64_t n_tok, int G) {
    const int D = src.D, ng = D / G;
    const int u = blockIdx.y;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // (token, group)
    if (idx >= n_tok * ng) return;
    const int64_t tau = idx / ng;
    const int gd = (int)(idx % ng);
    float mn = 1e30f, mx = -1e30f;
    for (int i = 0; i < G; ++i) {
        float v = src_load(src, u, tau, gd * G + i);
        mn = fminf(mn, v); mx = fmaxf(mx, v);
    }
    const float scale = group_scale(mn, mx);
        const float rcp = group_rcp(scale);
    const int64_t t = tok0 + tau;
    v_scales[(int64_t)u * max_tokens * ng + vmeta_index(t, gd, D, G)] = scale;
    v_zeros[(int64_t)u * max_tokens * ng + vmeta_index(t, gd, D, G)] = mn;
    uint8_t* dst = v_codes + (int64_t)u * max_tokens * (D / 4);
    for (int i = 0; i < G; i += 4) {
        uint32_t byte = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float q = code_magic<HALF_EVEN>(src_load(src, u, tau, gd * G + i + e), mn, scale, rcp);
            byte |= (__float_as_uint(q) & 3u) << (2 * e);
        }
        dst[vcode_offset(t, gd * (G / 4) + i / 4, D, G)] = (uint8_t)byte;
    }
}

// Values, fast path for D = 128, G = 32: four consecutive lanes share one
// (token, channel group); each lane owns 8 consecutive channels (one or two
// 128-bit loads), min/max finish with two xor-shuffles, a lane writes its two
// packed bytes, lane 0 of the four the scale and zero.  A warp covers two
// tokens, a CTA of 256 threads 16 tokens per iteration.
template <typename TR, typename TF, bool HALF_EVEN>
__global__ void __launch_bounds__(256)
flush_values_fast_kernel(TokenSource src, uint8_t* __restrict__ v_codes, float* __restrict__ v_scales,
                         float* __restrict__ v_zeros, int64_t max_tokens, int64_t tok0, int64_t n_tok) {
    constexpr int D = 128, G = 32, ITER = 4;             // 64 tokens = two value blocks per CTA
    // the blocks are assembled in shared memory (their bytes are permuted, see
    // vcode_offset) and leave with 128-bit stores
    __shared__ __align__(16) uint8_t s_codes[2 * 1024];
    __shared__ __align__(16) float s_scale[2 * 128];
    __shared__ __align__(16) float s_zero[2 * 128];
    const int u = blockIdx.y;
    const int lane16 = threadIdx.x & 15;                 // 16 lanes per token
    const int sub = lane16 & 3, gd = lane16 >> 2;
    const int64_t cta_tau0 = (int64_t)blockIdx.x * (ITER * 16);
    float v[ITER][8];
    int tl[ITER];                                        // token index inside the CTA's 64
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        tl[it] = it * 16 + (threadIdx.x >> 4);
        const int64_t tau = cta_tau0 + tl[it];
        if (tau < n_tok) {
            if (tau < src.res_len) {
                const int slot = (int)((src.res_start + tau) % src.R);
                Load8<TR>::run(reinterpret_cast<const TR*>(src.ring) + ((int64_t)u * src.R + slot) * D + lane16 * 8, v[it]);
            } else {
                Load8<TF>::run(reinterpret_cast<const TF*>(src.fresh) + (int64_t)u * src.unit_stride +
                                   (tau - src.res_len) * src.tok_stride + lane16 * 8, v[it]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[it][e] = 0.0f;
        }
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        float mn = 1e30f, mx = -1e30f;
#pragma unroll
        for (int e = 0; e < 8; ++e) { mn = fminf(mn, v[it][e]); mx = fmaxf(mx, v[it][e]); }
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 1)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 2)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float scale = group_scale(mn, mx);
        const float rcp = group_rcp(scale);
        uint32_t bytes = 0;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const float q0 = code_magic<HALF_EVEN>(v[it][4 * b + 0], mn, scale, rcp), q1 = code_magic<HALF_EVEN>(v[it][4 * b + 1], mn, scale, rcp);
            const float q2 = code_magic<HALF_EVEN>(v[it][4 * b + 2], mn, scale, rcp), q3 = code_magic<HALF_EVEN>(v[it][4 * b + 3], mn, scale, rcp);
            bytes |= pack4_magic(q0, q1, q2, q3) << (8 * b);
        }
        // offsets relative to the CTA's first token (a multiple of 64, so block aligned)
        s_codes[vcode_offset(tl[it], lane16 * 2, D, G)] = (uint8_t)bytes;
        s_codes[vcode_offset(tl[it], lane16 * 2 + 1, D, G)] = (uint8_t)(bytes >> 8);
        if (sub == 0) {
            const int mi = (int)vmeta_index(tl[it], gd, D, G);
            s_scale[mi] = scale; s_zero[mi] = mn;
        }
    }
    __syncthreads();
    // tok0 is a multiple of G and cta_tau0 of 64: whole blocks; a partial last CTA holds whole groups too
    const int64_t left = n_tok - cta_tau0;
    const int n_here = left < ITER * 16 ? (int)left : ITER * 16;        // multiple of 32
    const int64_t t_first = (int64_t)u * max_tokens + tok0 + cta_tau0;
    uint4* gc = reinterpret_cast<uint4*>(v_codes + t_first * (D / 4));
    float4* gs = reinterpret_cast<float4*>(v_scales + t_first * (D / G));
    float4* gz = reinterpret_cast<float4*>(v_zeros + t_first * (D / G));
    for (int i = threadIdx.x; i < n_here * 2; i += 256) gc[i] = reinterpret_cast<const uint4*>(s_codes)[i];
    for (int i = threadIdx.x; i < n_here; i += 256) {
        gs[i] = reinterpret_cast<const float4*>(s_scale)[i];
        gz[i] = reinterpret_cast<const float4*>(s_zero)[i];
    }
}

// ---- bulk prefill: groups cut straight out of the new tensor ----------------
// Keys for D = 128, G = 32, every token of the group in the new tensor: a warp
// owns 64 channels of one group, lane l channels 2l and 2l+1 of that half.  The
// 32 loads of a lane (one per token) are independent and each covers a full
// 128- or 256-byte piece of the token row across the warp, so nothing is staged
// and no barrier is needed; a lane keeps its group in registers, quantizes its
// two channels over the 32 tokens and writes its byte pairs (channels 2l and
// 2l+1 are neighbours in the key block) and scale/zero pairs directly.
// `fresh` points at the first token of the launch's first group; DENSE says
// that token rows follow each other without a gap (tok_stride == 128), which
// turns the 32 row offsets into immediates.
// grid = (ceil(2*n_groups / 4), units), 4 warps per CTA.
template <typename TF, bool HALF_EVEN, bool DENSE>
__global__ void __launch_bounds__(128)
flush_keys_direct_kernel(const TF* __restrict__ fresh, int64_t unit_stride, int64_t tok_stride_arg,
                         uint8_t* __restrict__ k_codes, float* __restrict__ k_scales,
                         float* __restrict__ k_zeros, int64_t max_groups, int64_t group0, int64_t n_groups) {
    constexpr int D = 128, G = 32, Q = 8;
    using P = Pair<TF>;
    const int64_t tok_stride = DENSE ? (int64_t)D : tok_stride_arg;
    const int u = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);      // (group, half)
    if (item >= 2 * n_groups) return;
    const int64_t gi = item >> 1;
    const int d = 64 * (int)(item & 1) + 2 * lane;
    const TF* src = fresh + (int64_t)u * unit_stride + gi * G * tok_stride + d;
    typename P::raw w[G];
#pragma unroll
    for (int t = 0; t < G; ++t) w[t] = P::load(src + t * tok_stride);
    typename P::acc lo = P::first(w[0]), hi = P::first(w[0]);
#pragma unroll
    for (int t = 1; t < G; ++t) { lo = P::lo(lo, w[t]); hi = P::hi(hi, w[t]); }
    float mn0, mn1, mx0, mx1;
    P::finish(lo, mn0, mn1);
    P::finish(hi, mx0, mx1);
    // the reference starts its reduction from +-1e30 (quant_tile.hpp:43-44)
    mn0 = fminf(mn0, 1e30f); mx0 = fmaxf(mx0, -1e30f); mn1 = fminf(mn1, 1e30f); mx1 = fmaxf(mx1, -1e30f);
    const float s0 = group_scale(mn0, mx0), s1 = group_scale(mn1, mx1);
    const float r0 = group_rcp(s0), r1 = group_rcp(s1);
    const int64_t g = group0 + gi;
    const int64_t meta = ((int64_t)u * max_groups + g) * D + d;
    *reinterpret_cast<float2*>(k_scales + meta) = make_float2(s0, s1);
    *reinterpret_cast<float2*>(k_zeros + meta) = make_float2(mn0, mn1);
    uint8_t* dst = k_codes + ((int64_t)u * max_groups + g) * (D * Q) + kblock_offset(d, 0, Q, 64);
    if (r0 != 0.0f && r1 != 0.0f) {
#pragma unroll
        for (int j = 0; j < Q; ++j) {
            float m0[4], m1[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float a, b;
                P::widen(w[4 * j + e], a, b);
                m0[e] = code_magic_rcp<HALF_EVEN>(a, mn0, s0, r0);
                m1[e] = code_magic_rcp<HALF_EVEN>(b, mn1, s1, r1);
            }
            *reinterpret_cast<uint16_t*>(dst + j * 64) =
                (uint16_t)(pack4_magic(m0[0], m0[1], m0[2], m0[3]) | (pack4_magic(m1[0], m1[1], m1[2], m1[3]) << 8));
        }
    } else {
        // a scale too large for a reciprocal (rare): plain divisions, the values
        // read again so that the register array is never indexed dynamically
#pragma unroll 1
        for (int j = 0; j < Q; ++j) {
            float m0[4], m1[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float a, b;
                P::widen(P::load(src + (4 * j + e) * tok_stride), a, b);
                m0[e] = code_magic<HALF_EVEN>(a, mn0, s0, r0);
                m1[e] = code_magic<HALF_EVEN>(b, mn1, s1, r1);
            }
            *reinterpret_cast<uint16_t*>(dst + j * 64) =
                (uint16_t)(pack4_magic(m0[0], m0[1], m0[2], m0[3]) | (pack4_magic(m1[0], m1[1], m1[2], m1[3]) << 8));
        }
    }
}

// Values for D = 128, G = 32, every token in the new tensor: a thread owns one
// (token, channel group) = 32 consecutive channels (no shuffles), thread
// 4*tl + gd of the CTA token tl of the CTA's 32.  With STAGED a warp first
// copies the 8 token rows of its threads to shared memory with loads that cover
// whole rows (a thread's own 128-bit loads would each touch 32 different lines),
// and every thread then reads its 32 channels from there; rows are padded by 16
// bytes so that both directions are free of bank conflicts for fp32.  The value
// block of the CTA is assembled in shared memory (planes padded to 68 words so
// that the byte stores of a warp spread over the banks) and leaves with 128-bit
// stores.  `fresh` points at the launch's first token, tok0 (a multiple of G)
// is its destination index; the grid covers whole groups.
template <typename TF, bool HALF_EVEN, bool STAGED>
__global__ void __launch_bounds__(128)
flush_values_direct_kernel(const TF* __restrict__ fresh, int64_t unit_stride, int64_t tok_stride,
                           uint8_t* __restrict__ v_codes, float* __restrict__ v_scales,
                           float* __restrict__ v_zeros, int64_t max_tokens, int64_t tok0) {
    constexpr int D = 128, G = 32, PLANE = 68;          // words per channel-group plane in shared memory
    constexpr int ROW_BYTES = G * (int)sizeof(TF), ROW_PITCH = ROW_BYTES + 16;
    __shared__ __align__(16) uint32_t s_codes[4 * PLANE];
    __shared__ __align__(16) float s_scale[128];
    __shared__ __align__(16) float s_zero[128];
    __shared__ __align__(16) uint8_t s_rows[STAGED ? 4 * 32 * ROW_PITCH : 16];
    const int u = blockIdx.y;
    const int tl = threadIdx.x >> 2, gd = threadIdx.x & 3;
    const int64_t cta_tau0 = (int64_t)blockIdx.x * G;
    const TF* src = fresh + (int64_t)u * unit_stride + (cta_tau0 + tl) * tok_stride + gd * G;
    Row32<TF> row;
    if (STAGED) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        uint8_t* mine = s_rows + warp * 32 * ROW_PITCH;
        constexpr int LANES_PER_TOKEN = D * (int)sizeof(TF) / 16;          // 32 (fp32) or 16 (bf16)
        constexpr int TOKENS_PER_LOAD = 32 / LANES_PER_TOKEN;
        const int piece = lane % LANES_PER_TOKEN;                          // 16-byte piece of the token row
        const uint8_t* tok = reinterpret_cast<const uint8_t*>(fresh + (int64_t)u * unit_stride + (cta_tau0 + 8 * warp + lane / LANES_PER_TOKEN) * tok_stride) + piece * 16;
#pragma unroll
        for (int k = 0; k < 8 / TOKENS_PER_LOAD; ++k) {
            const uint4 t = __ldg(reinterpret_cast<const uint4*>(tok + (int64_t)k * TOKENS_PER_LOAD * tok_stride * (int)sizeof(TF)));
            const int token = k * TOKENS_PER_LOAD + lane / LANES_PER_TOKEN;          // of the warp's 8
            const int r = 4 * token + piece * 16 / ROW_BYTES;                        // row = (token, channel group)
            *reinterpret_cast<uint4*>(mine + r * ROW_PITCH + (piece * 16) % ROW_BYTES) = t;
        }
        __syncwarp();
        row.load_staged(mine + lane * ROW_PITCH);
    } else {
        row.load(src);
    }
    float mn, mx;
    row.minmax(mn, mx);
    const float scale = group_scale(mn, mx);
    const float rcp = group_rcp(scale);
    // token tl = 16*kappa + 4*c + n: byte n of word gd*64 + kappa*32 + r*4 + c
    uint8_t* sc = reinterpret_cast<uint8_t*>(s_codes + gd * PLANE + (tl >> 4) * 32 + ((tl >> 2) & 3)) + (tl & 3);
    if (rcp != 0.0f) {
#pragma unroll
        for (int r = 0; r < G / 4; ++r) {
            float x[4];
            row.quad(r, x);
            sc[r * 16] = (uint8_t)pack4_magic(code_magic_rcp<HALF_EVEN>(x[0], mn, scale, rcp), code_magic_rcp<HALF_EVEN>(x[1], mn, scale, rcp),
                                              code_magic_rcp<HALF_EVEN>(x[2], mn, scale, rcp), code_magic_rcp<HALF_EVEN>(x[3], mn, scale, rcp));
        }
    } else {
        // a scale too large for a reciprocal (rare): plain divisions on re-read values
#pragma unroll 1
        for (int r = 0; r < G / 4; ++r) {
            float m[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
                m[e] = code_magic<HALF_EVEN>(load_as_float(src, sizeof(TF) == 2 ? KIVI_BF16 : KIVI_F32, 4 * r + e), mn, scale, rcp);
            sc[r * 16] = (uint8_t)pack4_magic(m[0], m[1], m[2], m[3]);
        }
    }
    const int mi = (int)vmeta_index(tl, gd, D, G);
    s_scale[mi] = scale; s_zero[mi] = mn;
    __syncthreads();
    const int64_t t_first = (int64_t)u * max_tokens + tok0 + cta_tau0;
    // 16-byte piece i of the block: plane i/16, piece i%16
    if (threadIdx.x < 64)
        reinterpret_cast<uint4*>(v_codes + t_first * (D / 4))[threadIdx.x] =
            *reinterpret_cast<const uint4*>(s_codes + (threadIdx.x >> 4) * PLANE + (threadIdx.x & 15) * 4);
    else if (threadIdx.x < 96)
        reinterpret_cast<float4*>(v_scales + t_first * (D / G))[threadIdx.x - 64] = reinterpret_cast<const float4*>(s_scale)[threadIdx.x - 64];
    else
        reinterpret_cast<float4*>(v_zeros + t_first * (D / G))[threadIdx.x - 96] = reinterpret_cast<const float4*>(s_zero)[threadIdx.x - 96];
}

// Copies virtual tokens [tau_from, tau_to) of the new tensor into their ring
// slots (slot = (res_start + tau) % R); tokens already in the ring stay put.
__global__ void __launch_bounds__(256)
ring_append_kernel(TokenSource src, void* __restrict__ k_ring, void* __restrict__ v_ring,
                   const void* __restrict__ fresh_v, int64_t unit_stride_v, int64_t tok_stride_v,
                   int64_t tau_from, int64_t tau_to) {
    const int D = src.D;
    const int u = blockIdx.y;
    const int64_t n = (tau_to - tau_from) * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tau = tau_from + i / D;
        const int d = (int)(i % D);
        const int slot = (int)((src.res_start + tau) % src.R);
        const int64_t o = ((int64_t)u * src.R + slot) * D + d;
        const int64_t tn = tau - src.res_len;
        float kv = load_as_float(src.fresh, src.fresh_dtype, (int64_t)u * src.unit_stride + tn * src.tok_stride + d);
        float vv = load_as_float(fresh_v, src.fresh_dtype, (int64_t)u * unit_stride_v + tn * tok_stride_v + d);
        store_from_float(k_ring, src.ring_dtype, o, kv);
        store_from_float(v_ring, src.ring_dtype, o, vv);
    }
}

// fp32 [units][T][D] keys and values: dequantized history then the window.
// A thread produces channels 4q .. 4q+3 of one token for both tensors: the four
// key codes sit in one aligned 32-bit word of the key block (the block's channel
// permutation keeps the two low bits), the four value codes in one byte, scales
// and zeros come as one 128-bit load (keys) or one scalar (values), and the
// results leave as two 128-bit stores.
__global__ void __launch_bounds__(256)
materialize_kernel(kivi_layer L, int64_t quant_len, int res_start, int res_len, int64_t t_begin,
                   float* __restrict__ k_out, float* __restrict__ v_out) {
    const int D = L.head_dim, G = L.group_size, Q = G / 4, W = D < 64 ? D : 64, ng = D / G, D4 = D / 4;
    const int u = blockIdx.y;
    const int64_t T = quant_len + res_len;
    const int64_t max_groups = L.max_tokens / G;
    const uint32_t n4 = (uint32_t)(T * D4);             // the host checks that this fits 31 bits
    const bool vec_out = ((reinterpret_cast<uintptr_t>(k_out) | reinterpret_cast<uintptr_t>(v_out)) & 15u) == 0;
    const bool vec_meta = ((reinterpret_cast<uintptr_t>(L.k_scales) | reinterpret_cast<uintptr_t>(L.k_zeros)) & 15u) == 0;
    const bool word_codes = (reinterpret_cast<uintptr_t>(L.k_codes) & 3u) == 0;
    for (uint32_t i = (uint32_t)t_begin * (uint32_t)D4 + blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += gridDim.x * blockDim.x) {                  // tokens t_begin .. T-1
        const uint32_t t = i / (uint32_t)D4;             // 32-bit index arithmetic: no 64-bit divisions per element
        const int d = (int)(i - t * (uint32_t)D4) * 4;
        float kv[4], vv[4];
        if (t < quant_len) {
            const uint32_t g = t / (uint32_t)G;
            const int tt = (int)(t - g * (uint32_t)G);
            const int j = tt >> 2, e = tt & 3;
            const int64_t gb = (int64_t)u * max_groups + g;
            const uint8_t* kc = L.k_codes + gb * (D * Q) + kblock_offset(d, j, Q, W);      // channels d..d+3: 4 adjacent bytes
            const uint32_t kw = word_codes ? *reinterpret_cast<const uint32_t*>(kc)
                                           : (uint32_t)kc[0] | ((uint32_t)kc[1] << 8) | ((uint32_t)kc[2] << 16) | ((uint32_t)kc[3] << 24);
            float ks[4], kz[4];
            if (vec_meta) {
                const float4 s4 = *reinterpret_cast<const float4*>(L.k_scales + gb * D + d);
                const float4 z4 = *reinterpret_cast<const float4*>(L.k_zeros + gb * D + d);
                ks[0] = s4.x; ks[1] = s4.y; ks[2] = s4.z; ks[3] = s4.w;
                kz[0] = z4.x; kz[1] = z4.y; kz[2] = z4.z; kz[3] = z4.w;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) { ks[c] = L.k_scales[gb * D + d + c]; kz[c] = L.k_zeros[gb * D + d + c]; }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
                kv[c] = dequant((float)((kw >> (8 * c + 2 * e)) & 3u), ks[c], kz[c]);
            const uint32_t vb = L.v_codes[(int64_t)u * L.max_tokens * D4 + vcode_offset(t, d >> 2, D, G)];
            const int64_t mi = (int64_t)u * L.max_tokens * ng + vmeta_index(t, d / G, D, G);
            const float vs = L.v_scales[mi], vz = L.v_zeros[mi];
#pragma unroll
            for (int c = 0; c < 4; ++c) vv[c] = dequant((float)((vb >> (2 * c)) & 3u), vs, vz);
        } else {
            int slot = res_start + (int)(t - quant_len);
            if (slot >= L.residual_cap) slot -= L.residual_cap;
            const int64_t o = ((int64_t)u * L.residual_cap + slot) * D + d;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                kv[c] = load_as_float(L.k_res, L.res_dtype, o + c);
                vv[c] = load_as_float(L.v_res, L.res_dtype, o + c);
            }
        }
        const int64_t o = (int64_t)u * T * D + (int64_t)i * 4;
        if (vec_out) {
            __stcs(reinterpret_cast<float4*>(k_out + o), make_float4(kv[0], kv[1], kv[2], kv[3]));
            __stcs(reinterpret_cast<float4*>(v_out + o), make_float4(vv[0], vv[1], vv[2], vv[3]));
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) { k_out[o + c] = kv[c]; v_out[o + c] = vv[c]; }
        }
    }
}

// Dequantized history for D = 128, G = 32: one warp per (unit, token group).
// Keys: lane l owns channels 4l .. 4l+3; its scales and zeros are two 128-bit
// loads for the whole group, each of its eight code words holds those channels
// for four tokens, and every store instruction of the warp writes one complete
// 512-byte token row.  Values: the lane dequantizes the eight words of the value
// block it loaded with two 128-bit loads (word (gd, kappa, r, c): natural byte
// 8*gd + r of tokens 16*kappa + 4*c + n); a store instruction writes 128-byte
// pieces of four token rows.  grid = (ceil(groups / 8), units), 8 warps.
__global__ void __launch_bounds__(256)
materialize_groups_kernel(kivi_layer L, int64_t n_groups, int64_t T,
                          float* __restrict__ k_out, float* __restrict__ v_out) {
    constexpr int D = 128, G = 32;
    const int u = blockIdx.y, lane = threadIdx.x & 31;
    const int64_t g = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (g >= n_groups) return;
    const int64_t max_groups = L.max_tokens / G;
    const int64_t gb = (int64_t)u * max_groups + g;
    float* ko = k_out + ((int64_t)u * T + g * G) * D;
    float* vo = v_out + ((int64_t)u * T + g * G) * D;
    {   // ---- keys
        const int d = 4 * lane;
        const float4 s4 = *reinterpret_cast<const float4*>(L.k_scales + gb * D + d);
        const float4 z4 = *reinterpret_cast<const float4*>(L.k_zeros + gb * D + d);
        const uint8_t* kc = L.k_codes + gb * (D * 8) + kblock_offset(d, 0, 8, 64);
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = *reinterpret_cast<const uint32_t*>(kc + j * 64);
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float4 r;
                r.x = dequant((float)((w[j] >> (2 * e)) & 3u), s4.x, z4.x);
                r.y = dequant((float)((w[j] >> (8 + 2 * e)) & 3u), s4.y, z4.y);
                r.z = dequant((float)((w[j] >> (16 + 2 * e)) & 3u), s4.z, z4.z);
                r.w = dequant((float)((w[j] >> (24 + 2 * e)) & 3u), s4.w, z4.w);
                __stcs(reinterpret_cast<float4*>(ko + (4 * j + e) * D + d), r);
            }
    }
    {   // ---- values
        const uint32_t* vb = reinterpret_cast<const uint32_t*>(L.v_codes + ((int64_t)u * L.max_tokens + g * G) * (D / 4));
        const float* vs = L.v_scales + ((int64_t)u * L.max_tokens + g * G) * 4;
        const float* vz = L.v_zeros + ((int64_t)u * L.max_tokens + g * G) * 4;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4 q4 = *reinterpret_cast<const uint4*>(vb + half * 128 + 4 * lane);
            const uint32_t w[4] = {q4.x, q4.y, q4.z, q4.w};
            // word 128*half + 4*lane + c: gd = 2*half + lane/16, kappa = (lane/8)%2, r = lane%8
            const int gd = 2 * half + (lane >> 4), kap = (lane >> 3) & 1, r = lane & 7;
            const int quad = 8 * gd + r;                                 // channels 4*quad .. 4*quad+3
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const int tt = 16 * kap + 4 * c + n;                 // token inside the group
                    const int row = 16 * kap + 4 * n + c;                // its scale / zero row
                    const float s = vs[row * 4 + gd], z = vz[row * 4 + gd];
                    const uint32_t b = (w[c] >> (8 * n)) & 0xffu;
                    float4 o;
                    o.x = dequant((float)(b & 3u), s, z);
                    o.y = dequant((float)((b >> 2) & 3u), s, z);
                    o.z = dequant((float)((b >> 4) & 3u), s, z);
                    o.w = dequant((float)(b >> 6), s, z);
                    __stcs(reinterpret_cast<float4*>(vo + tt * D + 4 * quad), o);
                }
        }
    }
}

// channel-major operator layout -> key blocks
__global__ void __launch_bounds__(256)
import_keys_kernel(kivi_layer L, const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                   const float* __restrict__ zeros, int64_t S) {
    const int D = L.head_dim, G = L.group_size, Q = G / 4, W = D < 64 ? D : 64;
    const int u = blockIdx.y;
    const int64_t n_groups = S / G, max_groups = L.max_tokens / G;
    const int64_t n = n_groups * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = i / D;
        const int d = (int)(i % D);
        const int64_t gb = (int64_t)u * max_groups + g;
        L.k_scales[gb * D + d] = scales[((int64_t)u * D + d) * n_groups + g];
        L.k_zeros[gb * D + d] = zeros[((int64_t)u * D + d) * n_groups + g];
        // operator bytes of this (channel, group): byte b = tokens 4b..4b+3
        const uint8_t* row = packed + ((int64_t)u * D + d) * (S / 4) + g * Q;
        for (int j = 0; j < Q; ++j) {
            const uint32_t byte = row[j];
            L.k_codes[gb * (D * Q) + kblock_offset(d, j, Q, W)] = (uint8_t)byte;
        }
    }
}

}  // namespace

int validate_layer(const kivi_layer* L) {
    KIVI_REQUIRE(L != nullptr, "layer is null");
    KIVI_REQUIRE(L->num_units > 0, "num_units must be positive, got %d", L->num_units);
    KIVI_REQUIRE(L->group_size >= 4 && L->group_size % 4 == 0,
                 "group_size (%d) must be >= 4 and divisible by 4", L->group_size);
    KIVI_REQUIRE(L->head_dim > 0 && L->head_dim % L->group_size == 0,
                 "head_dim (%d) must be divisible by group_size (%d)", L->head_dim, L->group_size);
    KIVI_REQUIRE(L->head_dim <= 64 || L->head_dim % 64 == 0,
                 "head_dim (%d) must be <= 64 or a multiple of 64", L->head_dim);
    KIVI_REQUIRE(L->head_dim <= 256, "head_dim (%d) above 256 is not supported", L->head_dim);
    KIVI_REQUIRE(L->group_size <= L->residual_cap,
                 "group_size (%d) must not exceed residual_length (%d)", L->group_size, L->residual_cap);
    KIVI_REQUIRE(L->max_tokens >= 0 && L->max_tokens % L->group_size == 0,
                 "max_tokens (%lld) must be a multiple of group_size", (long long)L->max_tokens);
    KIVI_REQUIRE(L->res_dtype == KIVI_F32 || L->res_dtype == KIVI_BF16, "res_dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(L->k_res && L->v_res, "residual ring pointers are null");
    if (L->max_tokens > 0)
        KIVI_REQUIRE(L->k_codes && L->k_scales && L->k_zeros && L->v_codes && L->v_scales && L->v_zeros,
                     "quantized store pointers are null");
    return KIVI_OK;
}

int validate_state(const kivi_layer* L, int64_t quant_len, int res_start, int res_len) {
    KIVI_REQUIRE(quant_len >= 0 && quant_len % L->group_size == 0 && quant_len <= L->max_tokens,
                 "quant_len (%lld) must be a multiple of group_size within max_tokens (%lld)",
                 (long long)quant_len, (long long)L->max_tokens);
    KIVI_REQUIRE(res_len >= 0 && res_len <= L->residual_cap, "res_len (%d) outside [0, %d]", res_len, L->residual_cap);
    KIVI_REQUIRE(res_start >= 0 && res_start < L->residual_cap, "res_start (%d) outside [0, %d)", res_start, L->residual_cap);
    return KIVI_OK;
}

}  // namespace kivi

using namespace kivi;

extern "C" int kivi_cache_plan(int64_t quant_len, int res_len, int n_new, int G, int R,
                               int* n_flush_groups, int64_t* quant_len_out, int* res_len_out) {
    KIVI_REQUIRE(G >= 4 && G % 4 == 0 && G <= R, "need 4 <= group_size <= residual_cap, group_size %% 4 == 0");
    KIVI_REQUIRE(quant_len >= 0 && res_len >= 0 && n_new >= 0, "negative length");
    const int64_t total = (int64_t)res_len + n_new;
    // while (len >= R) flush G  ==  floor((total - R) / G) + 1 flushes when total >= R
    const int64_t f = total >= R ? (total - R) / G + 1 : 0;
    if (n_flush_groups) *n_flush_groups = (int)f;
    if (quant_len_out) *quant_len_out = quant_len + f * G;
    if (res_len_out) *res_len_out = (int)(total - f * G);
    return KIVI_OK;
}

extern "C" int kivi_cache_update(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                                 const void* new_k, const void* new_v, int new_dtype,
                                 int64_t unit_stride_k, int64_t tok_stride_k,
                                 int64_t unit_stride_v, int64_t tok_stride_v, int n_new,
                                 int rounding, int64_t* quant_len_out, int* res_start_out,
                                 int* res_len_out, void* stream) {
    if (int rc = validate_layer(L)) return rc;
    if (int rc = validate_state(L, quant_len, res_start, res_len)) return rc;
    KIVI_REQUIRE(n_new > 0, "the forward pass produced no new tokens (n_new = %d)", n_new);
    KIVI_REQUIRE(new_k && new_v, "new_k / new_v are null");
    KIVI_REQUIRE(new_dtype == KIVI_F32 || new_dtype == KIVI_BF16, "new_dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(rounding == KIVI_ROUND_HALF_AWAY || rounding == KIVI_ROUND_HALF_EVEN, "unknown rounding %d", rounding);
    KIVI_REQUIRE(tok_stride_k >= L->head_dim && tok_stride_v >= L->head_dim, "token stride smaller than head_dim");
    const int G = L->group_size, R = L->residual_cap, D = L->head_dim;
    int f = 0, rl_out = 0;
    int64_t ql_out = 0;
    kivi_cache_plan(quant_len, res_len, n_new, G, R, &f, &ql_out, &rl_out);
    KIVI_REQUIRE(ql_out <= L->max_tokens, "quantized store overflow: need %lld tokens, capacity %lld",
                 (long long)ql_out, (long long)L->max_tokens);
    cudaStream_t st = (cudaStream_t)stream;
    int launches = 0;
    TokenSource sk{L->k_res, new_k, L->res_dtype, new_dtype, R, D, res_start, res_len, unit_stride_k, tok_stride_k};
    TokenSource sv{L->v_res, new_v, L->res_dtype, new_dtype, R, D, res_start, res_len, unit_stride_v, tok_stride_v};
    const int64_t max_groups = L->max_tokens / G;
    if (f > 0) {
        const int64_t group0 = quant_len / G;
        KIVI_REQUIRE(f <= 0x7fffffff && L->num_units <= 65535, "grid too large");
        const int threads = D >= 256 ? 256 : (D >= 128 ? 128 : (D >= 64 ? 64 : 32));
        const size_t smem = (size_t)D * G / 4;
        const bool he = rounding == KIVI_ROUND_HALF_EVEN;
        auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
        const int esz = elem_size(new_dtype);
        const bool fast_k = D == 128 && G == 32 && al16(new_k) && al16(L->k_res) && al16(L->k_codes) &&
                            al16(L->k_scales) && al16(L->k_zeros) &&
                            (unit_stride_k * esz) % 16 == 0 && (tok_stride_k * esz) % 16 == 0;
        // Groups that still contain ring tokens go through the kernels that read
        // the virtual sequence; the rest (a bulk prefill) is cut straight out of
        // the new tensor by the direct kernels.
        const int64_t g_ring = fast_k ? ((int64_t)(res_len + G - 1) / G < f ? (int64_t)(res_len + G - 1) / G : f) : f;
        if (g_ring > 0) {
            dim3 grid((unsigned)g_ring, (unsigned)L->num_units);
            if (fast_k) {
#define KIVI_FK(TR, TF)                                                                                              \
                do {                                                                                                 \
                    if (he) flush_keys_fast_kernel<TR, TF, true><<<grid, 128, 0, st>>>(sk, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0); \
                    else flush_keys_fast_kernel<TR, TF, false><<<grid, 128, 0, st>>>(sk, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0);   \
                } while (0)
                if (L->res_dtype == KIVI_F32 && new_dtype == KIVI_F32) KIVI_FK(float, float);
                else if (L->res_dtype == KIVI_F32) KIVI_FK(float, __nv_bfloat16);
                else if (new_dtype == KIVI_F32) KIVI_FK(__nv_bfloat16, float);
                else KIVI_FK(__nv_bfloat16, __nv_bfloat16);
#undef KIVI_FK
            } else if (G == 32) {
                if (he) flush_keys_kernel<32, true><<<grid, threads, smem, st>>>(sk, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0, G);
                else flush_keys_kernel<32, false><<<grid, threads, smem, st>>>(sk, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0, G);
            } else {
                if (he) flush_keys_kernel<0, true><<<grid, threads, smem, st>>>(sk, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0, G);
                else flush_keys_kernel<0, false><<<grid, threads, smem, st>>>(sk, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0, G);
            }
            KIVI_LAUNCH_OK();
            launches += 1;
        }
        if (g_ring < f) {
            const int64_t n_direct = f - g_ring;
            const int64_t first = g_ring * G - res_len;                       // index in the new tensor
            dim3 grid((unsigned)((2 * n_direct + 3) / 4), (unsigned)L->num_units);
#define KIVI_DK(TF)                                                                                                  \
            do {                                                                                                     \
                const TF* p = reinterpret_cast<const TF*>(new_k) + first * tok_stride_k;                             \
                if (tok_stride_k == D) {                                                                             \
                    if (he) flush_keys_direct_kernel<TF, true, true><<<grid, 128, 0, st>>>(p, unit_stride_k, tok_stride_k, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0 + g_ring, n_direct); \
                    else flush_keys_direct_kernel<TF, false, true><<<grid, 128, 0, st>>>(p, unit_stride_k, tok_stride_k, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0 + g_ring, n_direct);   \
                } else {                                                                                             \
                    if (he) flush_keys_direct_kernel<TF, true, false><<<grid, 128, 0, st>>>(p, unit_stride_k, tok_stride_k, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0 + g_ring, n_direct); \
                    else flush_keys_direct_kernel<TF, false, false><<<grid, 128, 0, st>>>(p, unit_stride_k, tok_stride_k, L->k_codes, L->k_scales, L->k_zeros, max_groups, group0 + g_ring, n_direct);   \
                }                                                                                                    \
            } while (0)
            if (new_dtype == KIVI_F32) KIVI_DK(float); else KIVI_DK(__nv_bfloat16);
#undef KIVI_DK
            KIVI_LAUNCH_OK();
            launches += 1;
        }
        const int64_t n_tok = (int64_t)f * G;
        const bool fast_v = D == 128 && G == 32 && al16(new_v) && al16(L->v_res) && al16(L->v_codes) &&
                            al16(L->v_scales) && al16(L->v_zeros) &&
                            (unit_stride_v * esz) % 16 == 0 && (tok_stride_v * esz) % 16 == 0;
        // tokens before t_ring (whole 64-token CTAs that may touch the ring) take the virtual-sequence kernels
        const int64_t t_ring = fast_v ? ((int64_t)(res_len + 63) / 64 * 64 < n_tok ? (int64_t)(res_len + 63) / 64 * 64 : n_tok) : n_tok;
        if (t_ring > 0) {
            if (fast_v) {
                dim3 gridv((unsigned)((t_ring + 63) / 64), (unsigned)L->num_units);
#define KIVI_FV(TR, TF)                                                                                              \
                do {                                                                                                 \
                    if (he) flush_values_fast_kernel<TR, TF, true><<<gridv, 256, 0, st>>>(sv, L->v_codes, L->v_scales, L->v_zeros, L->max_tokens, quant_len, t_ring); \
                    else flush_values_fast_kernel<TR, TF, false><<<gridv, 256, 0, st>>>(sv, L->v_codes, L->v_scales, L->v_zeros, L->max_tokens, quant_len, t_ring);   \
                } while (0)
                if (L->res_dtype == KIVI_F32 && new_dtype == KIVI_F32) KIVI_FV(float, float);
                else if (L->res_dtype == KIVI_F32) KIVI_FV(float, __nv_bfloat16);
                else if (new_dtype == KIVI_F32) KIVI_FV(__nv_bfloat16, float);
                else KIVI_FV(__nv_bfloat16, __nv_bfloat16);
#undef KIVI_FV
            } else {
                const int64_t items = n_tok * (D / G);
                dim3 gridv((unsigned)((items + 255) / 256), (unsigned)L->num_units);
                if (he) flush_values_kernel<true><<<gridv, 256, 0, st>>>(sv, L->v_codes, L->v_scales, L->v_zeros, L->max_tokens, quant_len, n_tok, G);
                else flush_values_kernel<false><<<gridv, 256, 0, st>>>(sv, L->v_codes, L->v_scales, L->v_zeros, L->max_tokens, quant_len, n_tok, G);
            }
            KIVI_LAUNCH_OK();
            launches += 1;
        }
        if (t_ring < n_tok) {
            const int64_t n_direct = n_tok - t_ring;
            dim3 gridv((unsigned)(n_direct / G), (unsigned)L->num_units);
// fp32 rows are staged through shared memory, bf16 rows are read directly
#define KIVI_STAGE(TF) (sizeof(TF) == 4 ? KIVI_STAGE_F32 : KIVI_STAGE_BF16)
#define KIVI_DV(TF)                                                                                                  \
            do {                                                                                                     \
                const TF* p = reinterpret_cast<const TF*>(new_v) + (t_ring - res_len) * tok_stride_v;                \
                if (he) flush_values_direct_kernel<TF, true, KIVI_STAGE(TF)><<<gridv, 128, 0, st>>>(p, unit_stride_v, tok_stride_v, L->v_codes, L->v_scales, L->v_zeros, L->max_tokens, quant_len + t_ring); \
                else flush_values_direct_kernel<TF, false, KIVI_STAGE(TF)><<<gridv, 128, 0, st>>>(p, unit_stride_v, tok_stride_v, L->v_codes, L->v_scales, L->v_zeros, L->max_tokens, quant_len + t_ring);   \
            } while (0)
            if (new_dtype == KIVI_F32) KIVI_DV(float); else KIVI_DV(__nv_bfloat16);
#undef KIVI_DV
#undef KIVI_STAGE
            KIVI_LAUNCH_OK();
            launches += 1;
        }
    }
    // tokens of the virtual sequence that stay: [f*G, res_len + n_new); those
    // with tau >= res_len come from the new tensor and must be copied in.
    const int64_t total = (int64_t)res_len + n_new;
    const int64_t tau_from = (int64_t)f * G > res_len ? (int64_t)f * G : res_len;
    if (tau_from < total) {
        const int64_t n = (total - tau_from) * D;
        unsigned bx = (unsigned)((n + 255) / 256);
        if (bx > 64) bx = 64;
        dim3 grid(bx, (unsigned)L->num_units);
        ring_append_kernel<<<grid, 256, 0, st>>>(sk, L->k_res, L->v_res, new_v, unit_stride_v, tok_stride_v, tau_from, total);
        KIVI_LAUNCH_OK();
        launches += 1;
    }
    if (quant_len_out) *quant_len_out = ql_out;
    if (res_start_out) *res_start_out = (int)((res_start + (int64_t)f * G) % R);
    if (res_len_out) *res_len_out = rl_out;
    note_launches(launches);
    return KIVI_OK;
}

extern "C" int kivi_cache_materialize(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                                      float* k_out, float* v_out, void* stream) {
    if (int rc = validate_layer(L)) return rc;
    if (int rc = validate_state(L, quant_len, res_start, res_len)) return rc;
    KIVI_REQUIRE(k_out && v_out, "output pointers are null");
    const int64_t n = (quant_len + res_len) * (L->head_dim / 4);
    if (n == 0) { note_launches(0); return KIVI_OK; }
    KIVI_REQUIRE(n < (1ll << 31), "too many tokens for one materialize call: %lld", (long long)(quant_len + res_len));
    cudaStream_t st = (cudaStream_t)stream;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    int launches = 0;
    int64_t t_begin = 0;
    // whole groups of the usual layer shape take the warp-per-group kernel; the
    // ring (and every other shape) the per-element one
    if (L->head_dim == 128 && L->group_size == 32 && quant_len > 0 && al16(k_out) && al16(v_out) && al16(L->k_codes) &&
        al16(L->k_scales) && al16(L->k_zeros) && al16(L->v_codes)) {
        const int64_t n_groups = quant_len / 32;
        dim3 grid((unsigned)((n_groups + 7) / 8), (unsigned)L->num_units);
        materialize_groups_kernel<<<grid, 256, 0, st>>>(*L, n_groups, quant_len + res_len, k_out, v_out);
        KIVI_LAUNCH_OK();
        ++launches;
        t_begin = quant_len;
    }
    const int64_t rest = (quant_len + res_len - t_begin) * (L->head_dim / 4);
    if (rest > 0) {
        unsigned bx = (unsigned)((rest + 255) / 256);
        if (bx > 4096) bx = 4096;
        dim3 grid(bx, (unsigned)L->num_units);
        materialize_kernel<<<grid, 256, 0, st>>>(*L, quant_len, res_start, res_len, t_begin, k_out, v_out);
        KIVI_LAUNCH_OK();
        ++launches;
    }
    note_launches(launches);
    return KIVI_OK;
}

extern "C" int kivi_cache_import_keys(const kivi_layer* L, const uint8_t* packed, const float* scales,
                                      const float* zeros, int64_t seq_len, void* stream) {
    if (int rc = validate_layer(L)) return rc;
    KIVI_REQUIRE(packed && scales && zeros, "packed / scales / zeros are null");
    KIVI_REQUIRE(seq_len > 0 && seq_len % L->group_size == 0 && seq_len <= L->max_tokens,
                 "seq_len (%lld) must be a positive multiple of group_size within max_tokens", (long long)seq_len);
    const int64_t n = seq_len / L->group_size * L->head_dim;
    unsigned bx = (unsigned)((n + 255) / 256);
    if (bx > 1024) bx = 1024;
    dim3 grid(bx, (unsigned)L->num_units);
    import_keys_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*L, packed, scales, zeros, seq_len);
    KIVI_LAUNCH_OK();
    note_launches(1);
    return KIVI_OK;
}
