// Flat-group 2-bit quantize / dequantize / round-trip operators (sm_100a).
//
// Each operator works on consecutive runs of `G` elements of the flat input,
// which is what both reference kernels do (keys per channel:
// src/csrc/kernels/quantize_kernels.cpp:39-51; values per token: :88-103, where
// base == gid*group_size because groups_per_token*group_size == head_dim).
//
// Fast kernel: LPG consecutive lanes share one group; every lane owns K*VEC
// consecutive elements, loaded as K 128-bit vectors (all loads of the CTA's
// tile are issued before any arithmetic).  min/max: in-lane, then xor-shuffles
// over the LPG lanes.  Codes are packed in registers, staged in shared memory
// together with the group's scale and zero, and the CTA writes the tile out
// with 128-bit stores.  HBM traffic per element: sizeof(T) read, 1/4 + 8/G
// bytes written.
// Generic kernel: one thread per group, two passes, for group sizes and
// alignments the fast kernel does not cover.
#include "kivi_common.cuh"

#include <type_traits>

namespace kivi {
namespace {

constexpr int kThreads = 256;
constexpr int kIter = 4;

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[4]) {
        float4 t = __ldg(reinterpret_cast<const float4*>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
        uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// MODE 0: write packed + scales + zeros.  MODE 1: write the round trip (fp32).
template <typename T, int LPG, int K, bool HALF_EVEN, int MODE>
__global__ void __launch_bounds__(kThreads)
group_quant_kernel(const T* __restrict__ in, uint8_t* __restrict__ packed,
                   float* __restrict__ scales, float* __restrict__ zeros,
                   float* __restrict__ rt_out, int64_t num_groups) {
    constexpr int VEC = Vec<T>::N;
    constexpr int EPL = K * VEC;            // elements per lane
    constexpr int G = EPL * LPG;            // group size
    constexpr int BPL = EPL / 4;            // packed bytes per lane
    constexpr int GPW = 32 / LPG;           // groups per warp per iteration
    constexpr int WARPS = kThreads / 32;
    constexpr int TILE_GROUPS = WARPS * GPW * kIter;
    constexpr int TILE_BYTES = TILE_GROUPS * (G / 4);

    __shared__ __align__(16) uint8_t s_codes[MODE == 0 ? TILE_BYTES : 16];
    __shared__ __align__(16) float s_scale[MODE == 0 ? TILE_GROUPS : 4];
    __shared__ __align__(16) float s_zero[MODE == 0 ? TILE_GROUPS : 4];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPG;
    const int64_t tile_g0 = (int64_t)blockIdx.x * TILE_GROUPS;

    float v[kIter][EPL];
    int lg[kIter];
#pragma unroll
    for (int it = 0; it < kIter; ++it) {
        lg[it] = (it * WARPS + warp) * GPW + lane / LPG;
        const int64_t g = tile_g0 + lg[it];
        if (g < num_groups) {
            const T* p = in + g * G + sub * EPL;
#pragma unroll
            for (int k = 0; k < K; ++k) {
                float t[VEC];
                Vec<T>::load(p + k * VEC, t);
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[it][k * VEC + e] = t[e];
            }
        } else {
#pragma unroll
            for (int e = 0; e < EPL; ++e) v[it][e] = 0.0f;
        }
    }

#pragma unroll
    for (int it = 0; it < kIter; ++it) {
        // min/max start at +-1e30f and ignore NaN (quant_tile.hpp:39-47)
        float mn = 1e30f, mx = -1e30f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            mn = fminf(mn, v[it][e]);
            mx = fmaxf(mx, v[it][e]);
        }
#pragma unroll
        for (int o = 1; o < LPG; o <<= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float scale = group_scale(mn, mx);
        const float rcp = group_rcp(scale);
        const int64_t g = tile_g0 + lg[it];
        // one branch per group, not per element: groups whose scale has no
        // reciprocal (>= 1e30) take the plain-division twin of the same code
        auto emit = [&](auto has_rcp) {
            constexpr bool RCP = decltype(has_rcp)::value;
            auto magic = [&](float x) {
                if constexpr (RCP) return code_magic_rcp<HALF_EVEN>(x, mn, scale, rcp);
                else return code_magic<HALF_EVEN>(x, mn, scale, rcp);
            };
            if (MODE == 0) {
                uint32_t bytes[(BPL + 3) / 4] = {};
#pragma unroll
                for (int b = 0; b < BPL; ++b) {
                    const uint32_t byte = pack4_magic(magic(v[it][4 * b + 0]), magic(v[it][4 * b + 1]),
                                                      magic(v[it][4 * b + 2]), magic(v[it][4 * b + 3]));
                    bytes[b / 4] |= byte << (8 * (b % 4));
                }
                uint8_t* dst = s_codes + lg[it] * (G / 4) + sub * BPL;
                if (BPL == 1) *dst = (uint8_t)bytes[0];
                else if (BPL == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)bytes[0];
                else {
#pragma unroll
                    for (int w = 0; w < BPL / 4; ++w) reinterpret_cast<uint32_t*>(dst)[w] = bytes[w];
                }
                if (sub == 0) { s_scale[lg[it]] = scale; s_zero[lg[it]] = mn; }
            } else if (g < num_groups) {
                float* o = rt_out + g * G + sub * EPL;
#pragma unroll
                for (int k = 0; k < EPL / 4; ++k) {
                    float4 r;
                    r.x = dequant(__fsub_rn(magic(v[it][4 * k + 0]), 8388608.0f), scale, mn);
                    r.y = dequant(__fsub_rn(magic(v[it][4 * k + 1]), 8388608.0f), scale, mn);
                    r.z = dequant(__fsub_rn(magic(v[it][4 * k + 2]), 8388608.0f), scale, mn);
                    r.w = dequant(__fsub_rn(magic(v[it][4 * k + 3]), 8388608.0f), scale, mn);
                    reinterpret_cast<float4*>(o)[k] = r;
                }
            }
        };
        if (rcp != 0.0f) emit(std::true_type{}); else emit(std::false_type{});
    }
    if (MODE != 0) return;
    __syncthreads();

    int64_t left = num_groups - tile_g0;
    const int valid = left < TILE_GROUPS ? (int)left : TILE_GROUPS;
    const int valid_bytes = valid * (G / 4);
    uint8_t* gp = packed + tile_g0 * (G / 4);
    for (int i = threadIdx.x * 16; i < valid_bytes; i += kThreads * 16) {
        if (i + 16 <= valid_bytes) {
            *reinterpret_cast<uint4*>(gp + i) = *reinterpret_cast<const uint4*>(s_codes + i);
        } else {
            for (int b = i; b < valid_bytes; ++b) gp[b] = s_codes[b];
        }
    }
    float* gs = scales + tile_g0;
    float* gz = zeros + tile_g0;
    for (int i = threadIdx.x * 4; i < valid; i += kThreads * 4) {
        if (i + 4 <= valid) {
            *reinterpret_cast<float4*>(gs + i) = *reinterpret_cast<const float4*>(s_scale + i);
            *reinterpret_cast<float4*>(gz + i) = *reinterpret_cast<const float4*>(s_zero + i);
        } else {
            for (int b = i; b < valid; ++b) { gs[b] = s_scale[b]; gz[b] = s_zero[b]; }
        }
    }
}

// One thread per group, any G % 4 == 0, any alignment.
template <bool HALF_EVEN, int MODE>
__global__ void __launch_bounds__(kThreads)
group_quant_generic_kernel(const void* __restrict__ in, int in_dtype, uint8_t* __restrict__ packed,
                           float* __restrict__ scales, float* __restrict__ zeros,
                           float* __restrict__ rt_out, int64_t num_groups, int G) {
    const int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (g >= num_groups) return;
    const int64_t base = g * G;
    float mn = 1e30f, mx = -1e30f;
    for (int i = 0; i < G; ++i) {
        float x = load_as_float(in, in_dtype, base + i);
        mn = fminf(mn, x);
        mx = fmaxf(mx, x);
    }
    const float scale = group_scale(mn, mx);
        const float rcp = group_rcp(scale);
    if (MODE == 0) {
        scales[g] = scale;
        zeros[g] = mn;
        for (int i = 0; i < G; i += 4) {
            uint32_t byte = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float q = code_magic<HALF_EVEN>(load_as_float(in, in_dtype, base + i + j), mn, scale, rcp);
                byte |= (__float_as_uint(q) & 3u) << (2 * j);
            }
            packed[g * (G / 4) + i / 4] = (uint8_t)byte;
        }
    } else {
        for (int i = 0; i < G; ++i) {
            float q = code_of<HALF_EVEN>(load_as_float(in, in_dtype, base + i), mn, scale, rcp);
            rt_out[base + i] = dequant(q, scale, mn);
        }
    }
}

// bf16 input, G = 32*NR (32, 64 or 128), quantize only: one thread per group.
// The group arrives as independent 128-bit loads and stays in registers as
// loaded (min/max on bf16 pairs, widened only when quantized); the packed bytes
// leave as 64- or 128-bit stores, so a warp writes contiguous runs of codes,
// scales and zeros: no shuffles, no staging, no barrier.
template <bool HALF_EVEN, int NR>
__global__ void __launch_bounds__(kThreads)
group_quant_bf16_rows_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ packed,
                             float* __restrict__ scales, float* __restrict__ zeros, int64_t num_groups) {
    constexpr int G = 32 * NR;
    const int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (g >= num_groups) return;
    const __nv_bfloat16* src = in + g * G;
    Row32<__nv_bfloat16> row[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) row[k].load(src + 32 * k);
    float mn = 1e30f, mx = -1e30f;
#pragma unroll
    for (int k = 0; k < NR; ++k) {
        float a, b;
        row[k].minmax(a, b);
        mn = fminf(mn, a); mx = fmaxf(mx, b);
    }
    const float scale = group_scale(mn, mx);
    const float rcp = group_rcp(scale);
    uint32_t w[2 * NR];
#pragma unroll
    for (int i = 0; i < 2 * NR; ++i) w[i] = 0u;
    if (rcp != 0.0f) {
#pragma unroll
        for (int k = 0; k < NR; ++k)
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                float x[4];
                row[k].quad(r, x);
                w[2 * k + (r >> 2)] |= pack4_magic(code_magic_rcp<HALF_EVEN>(x[0], mn, scale, rcp), code_magic_rcp<HALF_EVEN>(x[1], mn, scale, rcp),
                                                   code_magic_rcp<HALF_EVEN>(x[2], mn, scale, rcp), code_magic_rcp<HALF_EVEN>(x[3], mn, scale, rcp))
                                       << (8 * (r & 3));
            }
        if (NR == 1) {
            *reinterpret_cast<uint2*>(packed + g * 8) = make_uint2(w[0], w[1]);
        } else {
#pragma unroll
            for (int i = 0; i < NR / 2; ++i)
                reinterpret_cast<uint4*>(packed + g * (G / 4))[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
    } else {
        // a scale too large for a reciprocal (rare): plain divisions on re-read values
        for (int b = 0; b < G / 4; ++b) {
            float m[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) m[e] = code_magic<HALF_EVEN>(__bfloat162float(src[4 * b + e]), mn, scale, rcp);
            packed[g * (G / 4) + b] = (uint8_t)pack4_magic(m[0], m[1], m[2], m[3]);
        }
    }
    scales[g] = scale;
    zeros[g] = mn;
}

template <int NR>
int launch_bf16_rows(const void* in, uint8_t* packed, float* scales, float* zeros, int64_t num_groups, int rounding,
                     cudaStream_t st) {
    const int64_t blocks = (num_groups + kThreads - 1) / kThreads;
    KIVI_REQUIRE(blocks <= 0x7fffffffLL, "too many groups for one launch: %lld", (long long)num_groups);
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(in);
    if (rounding == KIVI_ROUND_HALF_EVEN)
        group_quant_bf16_rows_kernel<true, NR><<<(unsigned)blocks, kThreads, 0, st>>>(p, packed, scales, zeros, num_groups);
    else
        group_quant_bf16_rows_kernel<false, NR><<<(unsigned)blocks, kThreads, 0, st>>>(p, packed, scales, zeros, num_groups);
    KIVI_LAUNCH_OK();
    note_launches(1);
    return KIVI_OK;
}

// Dequantize: one packed byte -> one float4 (dequantize_kernels.cpp:50-61).  The
// kernel is bound by its 16-bytes-per-input-byte output stream, so what matters
// is how many stores a thread has in flight: a CTA takes a tile of
// kDqUnroll * kThreads consecutive bytes, a thread the bytes t, t + kThreads, ...
// of it (every load and every 128-bit store of a warp is one contiguous run), all
// of a thread's loads are issued before its first store.
constexpr int kDqUnroll = 8;

__device__ __forceinline__ float4 dequant_byte(uint32_t p, float s, float z) {
    // code c as a float: the two bits dropped into the mantissa of 2^23, minus 2^23
    float4 r;
    r.x = dequant(__fsub_rn(__uint_as_float(0x4B000000u | (p & 3u)), 8388608.0f), s, z);
    r.y = dequant(__fsub_rn(__uint_as_float(0x4B000000u | ((p >> 2) & 3u)), 8388608.0f), s, z);
    r.z = dequant(__fsub_rn(__uint_as_float(0x4B000000u | ((p >> 4) & 3u)), 8388608.0f), s, z);
    r.w = dequant(__fsub_rn(__uint_as_float(0x4B000000u | (p >> 6)), 8388608.0f), s, z);
    return r;
}

__global__ void __launch_bounds__(kThreads)
group_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                     const float* __restrict__ zeros, float* __restrict__ out,
                     int64_t total_bytes, int bytes_per_group, int group_shift, bool vec_ok) {
    const int64_t tile = (int64_t)kDqUnroll * kThreads;
    for (int64_t b0 = (int64_t)blockIdx.x * tile; b0 < total_bytes; b0 += (int64_t)gridDim.x * tile) {
        uint32_t p[kDqUnroll];
        float s[kDqUnroll], z[kDqUnroll];
#pragma unroll
        for (int k = 0; k < kDqUnroll; ++k) {
            const int64_t b = b0 + (int64_t)k * kThreads + threadIdx.x;
            if (b < total_bytes) {
                // group of this byte: a shift for power-of-two groups (no 64-bit division per element)
                const int64_t g = group_shift >= 0 ? (b >> group_shift) : b / bytes_per_group;
                p[k] = __ldg(packed + b);
                s[k] = __ldg(scales + g);
                z[k] = __ldg(zeros + g);
            }
        }
#pragma unroll
        for (int k = 0; k < kDqUnroll; ++k) {
            const int64_t b = b0 + (int64_t)k * kThreads + threadIdx.x;
            if (b < total_bytes) {
                const float4 r = dequant_byte(p[k], s[k], z[k]);
                if (vec_ok) {
                    __stcs(reinterpret_cast<float4*>(out) + b, r);
                } else {
                    out[4 * b] = r.x; out[4 * b + 1] = r.y; out[4 * b + 2] = r.z; out[4 * b + 3] = r.w;
                }
            }
        }
    }
}

template <typename T, int LPG, int K>
int launch_fast(const void* in, uint8_t* packed, float* scales, float* zeros, float* rt,
                int64_t num_groups, int rounding, int mode, cudaStream_t st) {
    constexpr int GPW = 32 / LPG;
    constexpr int TILE_GROUPS = (kThreads / 32) * GPW * kIter;
    const int64_t blocks = (num_groups + TILE_GROUPS - 1) / TILE_GROUPS;
    KIVI_REQUIRE(blocks <= 0x7fffffffLL, "too many groups for one launch: %lld", (long long)num_groups);
    const T* p = reinterpret_cast<const T*>(in);
    dim3 grid((unsigned)blocks), block(kThreads);
    if (mode == 0) {
        if (rounding == KIVI_ROUND_HALF_EVEN)
            group_quant_kernel<T, LPG, K, true, 0><<<grid, block, 0, st>>>(p, packed, scales, zeros, rt, num_groups);
        else
            group_quant_kernel<T, LPG, K, false, 0><<<grid, block, 0, st>>>(p, packed, scales, zeros, rt, num_groups);
    } else {
        if (rounding == KIVI_ROUND_HALF_EVEN)
            group_quant_kernel<T, LPG, K, true, 1><<<grid, block, 0, st>>>(p, packed, scales, zeros, rt, num_groups);
        else
            group_quant_kernel<T, LPG, K, false, 1><<<grid, block, 0, st>>>(p, packed, scales, zeros, rt, num_groups);
    }
    KIVI_LAUNCH_OK();
    note_launches(1);
    return KIVI_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// mode 0: quantize, mode 1: round trip
int run_group_quant(const void* in, int in_dtype, uint8_t* packed, float* scales, float* zeros,
                    float* rt, int64_t num_groups, int G, int rounding, int mode,
                    cudaStream_t st) {
    KIVI_REQUIRE(in != nullptr, "input is null");
    KIVI_REQUIRE(in_dtype == KIVI_F32 || in_dtype == KIVI_BF16, "input dtype must be KIVI_F32 or KIVI_BF16, got %d", in_dtype);
    KIVI_REQUIRE(rounding == KIVI_ROUND_HALF_AWAY || rounding == KIVI_ROUND_HALF_EVEN, "unknown rounding %d", rounding);
    KIVI_REQUIRE(G > 0 && G % 4 == 0, "group_size must be positive and divisible by 4, got %d", G);
    KIVI_REQUIRE(num_groups > 0, "input must be non-empty");
    if (mode == 0) KIVI_REQUIRE(packed && scales && zeros, "output, scales and zeros must be non-null");
    else KIVI_REQUIRE(rt != nullptr, "output is null");

    const bool al = aligned16(in) && (mode == 0 ? (aligned16(packed) && aligned16(scales) && aligned16(zeros)) : aligned16(rt));
    if (al) {
        if (in_dtype == KIVI_F32) {
            switch (G) {
                case 16: return launch_fast<float, 4, 1>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                case 32: return launch_fast<float, 4, 2>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                case 64: return launch_fast<float, 8, 2>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                case 128: return launch_fast<float, 16, 2>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                default: break;
            }
        } else {
            if (mode == 0) {
                if (G == 32) return launch_bf16_rows<1>(in, packed, scales, zeros, num_groups, rounding, st);
                if (G == 64) return launch_bf16_rows<2>(in, packed, scales, zeros, num_groups, rounding, st);
                if (G == 128) return launch_bf16_rows<4>(in, packed, scales, zeros, num_groups, rounding, st);
            }
            switch (G) {
                case 16: return launch_fast<__nv_bfloat16, 2, 1>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                case 32: return launch_fast<__nv_bfloat16, 4, 1>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                case 64: return launch_fast<__nv_bfloat16, 8, 1>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                case 128: return launch_fast<__nv_bfloat16, 16, 1>(in, packed, scales, zeros, rt, num_groups, rounding, mode, st);
                default: break;
            }
        }
    }
    const int64_t blocks = (num_groups + kThreads - 1) / kThreads;
    KIVI_REQUIRE(blocks <= 0x7fffffffLL, "too many groups for one launch: %lld", (long long)num_groups);
    dim3 grid((unsigned)blocks), block(kThreads);
    if (mode == 0) {
        if (rounding == KIVI_ROUND_HALF_EVEN)
            group_quant_generic_kernel<true, 0><<<grid, block, 0, st>>>(in, in_dtype, packed, scales, zeros, rt, num_groups, G);
        else
            group_quant_generic_kernel<false, 0><<<grid, block, 0, st>>>(in, in_dtype, packed, scales, zeros, rt, num_groups, G);
    } else {
        if (rounding == KIVI_ROUND_HALF_EVEN)
            group_quant_generic_kernel<true, 1><<<grid, block, 0, st>>>(in, in_dtype, packed, scales, zeros, rt, num_groups, G);
        else
            group_quant_generic_kernel<false, 1><<<grid, block, 0, st>>>(in, in_dtype, packed, scales, zeros, rt, num_groups, G);
    }
    KIVI_LAUNCH_OK();
    note_launches(1);
    return KIVI_OK;
}

int run_group_dequant(const uint8_t* packed, const float* scales, const float* zeros, float* out,
                      int64_t num_groups, int G, cudaStream_t st) {
    KIVI_REQUIRE(packed && scales && zeros && out, "input, scales, zeros and output must be non-null");
    KIVI_REQUIRE(G > 0 && G % 4 == 0, "group_size must be positive and divisible by 4, got %d", G);
    KIVI_REQUIRE(num_groups > 0, "scales must be non-empty");
    const int64_t total_bytes = num_groups * (G / 4);
    int64_t blocks = (total_bytes + (int64_t)kDqUnroll * kThreads - 1) / ((int64_t)kDqUnroll * kThreads);
    const int64_t cap = (int64_t)num_sms() * 32;
    if (blocks > cap) blocks = cap;
    int shift = -1;
    for (int k = 0; k < 31; ++k) if ((G / 4) == (1 << k)) shift = k;
    group_dequant_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(packed, scales, zeros, out, total_bytes, G / 4, shift, aligned16(out));
    KIVI_LAUNCH_OK();
    note_launches(1);
    return KIVI_OK;
}

}  // namespace kivi
