// Shared host/device helpers of libkivi_cuda (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "kivi_cuda.h"

namespace kivi {

// ---- error plumbing ---------------------------------------------------------
void set_error(const char* fmt, ...);
void note_launches(int n);
int num_sms();

#define KIVI_REQUIRE(cond, ...)                        \
    do {                                               \
        if (!(cond)) {                                 \
            ::kivi::set_error(__VA_ARGS__);            \
            return KIVI_ERR_INVALID_ARGUMENT;          \
        }                                              \
    } while (0)

#define KIVI_CUDA_OK(expr)                                                          \
    do {                                                                            \
        cudaError_t e_ = (expr);                                                    \
        if (e_ != cudaSuccess) {                                                    \
            ::kivi::set_error("%s failed: %s", #expr, cudaGetErrorString(e_));      \
            return KIVI_ERR_CUDA;                                                   \
        }                                                                           \
    } while (0)

#define KIVI_LAUNCH_OK()  KIVI_CUDA_OK(cudaGetLastError())

// ---- arithmetic that must match the reference bit for bit ------------------
// scale = (max - min) / 3.0f + 1e-10f      (quantize_kernels.cpp:46)
// The division by 3 is the correctly rounded quotient from a multiply and two
// FMAs (q0 = RN(r * RN(1/3)), e = r - 3*q0 exact, RN(q0 + e * RN(1/3))); checked
// equal to r / 3.0f for every mantissa at 18 exponents spanning the range and
// for every subnormal r.  An infinite range takes the plain division.
__device__ __forceinline__ float group_scale(float mn, float mx) {
    const float r = __fsub_rn(mx, mn);
    const float third = 0.3333333432674407958984375f;    // RN(1/3)
    float q;
    if (r <= 3.0e38f) {
        const float q0 = __fmul_rn(r, third);
        const float e = __fmaf_rn(-3.0f, q0, r);
        q = __fmaf_rn(e, third, q0);
    } else {
        q = __fdiv_rn(r, 3.0f);
    }
    return __fadd_rn(q, 1e-10f);
}

// Per-group reciprocal for the exact division below; 0 selects the plain IEEE
// division (scales so large that 1/scale would be subnormal).
__device__ __forceinline__ float group_rcp(float scale) {
    return scale < 1e30f ? __frcp_rn(scale) : 0.0f;
}

// q = clamp(round((x - min) / scale), 0, 3)   (quant_tile.hpp:61-66), returned
// as the float 2^23 + q, whose two lowest mantissa bits are the code.
//
// The quotient t is the correctly rounded IEEE quotient: with r = RN(1/scale),
// q0 = RN(a*r), e = a - scale*q0 (exact in an FMA), RN(q0 + e*r) equals
// RN(a/scale) (Markstein's correction step; checked against IEEE division on
// 6e8 samples including tie-heavy bf16 data).
//
// Rounding without a round instruction: 0 <= t <= 3.0000005 because
// a <= RN(max - min) and scale >= RN(RN(max - min) / 3), so the clamp never
// binds and adding 2^23 leaves round(t) in the mantissa.  Half to even is the
// add's own rounding.  Half away from zero is floor(t + 0.5): the first add
// rounds down, which cannot cross an integer n (n is representable, so
// RD(t + 0.5) >= n exactly when t + 0.5 >= n), the second add rounds down to
// an integer.
template <bool HALF_EVEN>
__device__ __forceinline__ float code_magic(float x, float mn, float scale, float rcp) {
    const float a = __fsub_rn(x, mn);
    float t;
    if (rcp != 0.0f) {
        const float q0 = __fmul_rn(a, rcp);
        const float e = __fmaf_rn(-scale, q0, a);
        t = __fmaf_rn(e, rcp, q0);
    } else {
        t = __fdiv_rn(a, scale);
    }
    if (HALF_EVEN) return __fadd_rn(t, 8388608.0f);
    return __fadd_rd(__fadd_rd(t, 0.5f), 8388608.0f);
}

// code_magic for a group whose reciprocal exists (rcp != 0): no branch per element
template <bool HALF_EVEN>
__device__ __forceinline__ float code_magic_rcp(float x, float mn, float scale, float rcp) {
    const float a = __fsub_rn(x, mn);
    const float q0 = __fmul_rn(a, rcp);
    const float e = __fmaf_rn(-scale, q0, a);
    const float t = __fmaf_rn(e, rcp, q0);
    if (HALF_EVEN) return __fadd_rn(t, 8388608.0f);
    return __fadd_rd(__fadd_rd(t, 0.5f), 8388608.0f);
}

// the code as a float in {0, 1, 2, 3}
template <bool HALF_EVEN>
__device__ __forceinline__ float code_of(float x, float mn, float scale, float rcp) {
    return __fsub_rn(code_magic<HALF_EVEN>(x, mn, scale, rcp), 8388608.0f);
}

// byte q0 | q1<<2 | q2<<4 | q3<<6 (quant_tile.hpp:61-68) from four code_magic
// values: the 2^23 offsets only reach bits 8 and up of the integer sum.
__device__ __forceinline__ uint32_t pack4_magic(float m0, float m1, float m2, float m3) {
    const uint32_t b = ((__float_as_uint(m3) * 4u + __float_as_uint(m2)) * 4u + __float_as_uint(m1)) * 4u + __float_as_uint(m0);
    return b & 0xffu;
}

// out = float(q) * scale + zero with a separate multiply and add
// (dequantize_kernels.cpp:23-25)
__device__ __forceinline__ float dequant(float q, float scale, float zero) {
    return __fadd_rn(__fmul_rn(q, scale), zero);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t hi16) {
    return __uint_as_float(hi16 << 16);
}

__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
    if (dtype == KIVI_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_from_float(void* p, int dtype, int64_t i, float v) {
    if (dtype == KIVI_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p)[i] = v;
}

// ---- groups kept in registers as loaded -----------------------------------------
// Two neighbouring elements kept as loaded (one 32-bit word for bf16, so a
// lane's group costs half the registers), widened to fp32 only where used.
// Minimum and maximum of bf16 pairs run on both halves at once; they are exact
// in any format, and which zero wins a tie between -0 and +0 does not change a
// code or a dequantized value's numeric value.
template <typename T> struct Pair;
template <> struct Pair<float> {
    using raw = float2;
    using acc = float2;
    __device__ static raw load(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
    __device__ static void widen(raw w, float& a, float& b) { a = w.x; b = w.y; }
    __device__ static acc first(raw w) { return w; }
    __device__ static acc lo(acc m, raw w) { return make_float2(fminf(m.x, w.x), fminf(m.y, w.y)); }
    __device__ static acc hi(acc m, raw w) { return make_float2(fmaxf(m.x, w.x), fmaxf(m.y, w.y)); }
    __device__ static void finish(acc m, float& a, float& b) { a = m.x; b = m.y; }
};
template <> struct Pair<__nv_bfloat16> {
    using raw = uint32_t;
    using acc = __nv_bfloat162;
    __device__ static raw load(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }
    __device__ static void widen(raw w, float& a, float& b) { a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xffff0000u); }
    __device__ static acc first(raw w) { return *reinterpret_cast<const __nv_bfloat162*>(&w); }
    __device__ static acc lo(acc m, raw w) { return __hmin2(m, *reinterpret_cast<const __nv_bfloat162*>(&w)); }
    __device__ static acc hi(acc m, raw w) { return __hmax2(m, *reinterpret_cast<const __nv_bfloat162*>(&w)); }
    __device__ static void finish(acc m, float& a, float& b) { widen(*reinterpret_cast<const uint32_t*>(&m), a, b); }
};

// The 32 channels of one (token, channel group) kept as loaded: four 128-bit
// words for bf16, eight for fp32.
template <typename T> struct Row32;
template <> struct Row32<float> {
    float4 v[8];
    __device__ void load(const float* p) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = __ldg(reinterpret_cast<const float4*>(p) + k);
    }
    __device__ void load_staged(const uint8_t* p) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = reinterpret_cast<const float4*>(p)[k];
    }
    __device__ void minmax(float& mn, float& mx) const {
        mn = 1e30f; mx = -1e30f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            mn = fminf(fminf(mn, v[k].x), fminf(v[k].y, fminf(v[k].z, v[k].w)));
            mx = fmaxf(fmaxf(mx, v[k].x), fmaxf(v[k].y, fmaxf(v[k].z, v[k].w)));
        }
    }
    // channels 4r .. 4r+3
    __device__ void quad(int r, float (&x)[4]) const { x[0] = v[r].x; x[1] = v[r].y; x[2] = v[r].z; x[3] = v[r].w; }
};
template <> struct Row32<__nv_bfloat16> {
    uint32_t w[16];
    __device__ void load(const __nv_bfloat16* p) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint4 t = __ldg(reinterpret_cast<const uint4*>(p) + k);
            w[4 * k] = t.x; w[4 * k + 1] = t.y; w[4 * k + 2] = t.z; w[4 * k + 3] = t.w;
        }
    }
    __device__ void load_staged(const uint8_t* p) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint4 t = reinterpret_cast<const uint4*>(p)[k];
            w[4 * k] = t.x; w[4 * k + 1] = t.y; w[4 * k + 2] = t.z; w[4 * k + 3] = t.w;
        }
    }
    __device__ void minmax(float& mn, float& mx) const {
        using P = Pair<__nv_bfloat16>;
        P::acc lo = P::first(w[0]), hi = P::first(w[0]);
#pragma unroll
        for (int k = 1; k < 16; ++k) { lo = P::lo(lo, w[k]); hi = P::hi(hi, w[k]); }
        float a, b;
        P::finish(lo, a, b); mn = fminf(fminf(a, b), 1e30f);
        P::finish(hi, a, b); mx = fmaxf(fmaxf(a, b), -1e30f);
    }
    __device__ void quad(int r, float (&x)[4]) const {
        Pair<__nv_bfloat16>::widen(w[2 * r], x[0], x[1]);
        Pair<__nv_bfloat16>::widen(w[2 * r + 1], x[2], x[3]);
    }
};

// ---- key block layout --------------------------------------------------------
// Byte offset inside one key block of the codes of channel d, token quad j
// (tokens 4j .. 4j+3 of the group in bits 0-1, 2-3, 4-5, 6-7; 0 <= j < Q = G/4);
// W = min(D, 64).  Within a 64-channel half-row the two 2-bit fields (d>>2)&3
// and (d>>4)&3 of the channel index are swapped, so that a 16-byte piece of a
// row holds four 4-channel words that are 16 channels apart: the tensor-core
// kernel gives each lane one such piece and then reads the matching scales
// without bank conflicts.
__host__ __device__ __forceinline__ int kblock_offset(int d, int j, int Q, int W) {
    int dl = d % W;
    if (W == 64) dl = (dl & 3) | (((dl >> 4) & 3) << 2) | (((dl >> 2) & 3) << 4);
    return (d / W) * Q * W + j * W + dl;
}

// ---- value layout ---------------------------------------------------------------
// Values keep the reference's per-token rows (byte b of token t = channels
// 4b..4b+3, quantize_kernels.hpp:55-60) except for D = 128, G = 32, where the
// 32 rows of a token group are re-laid inside their own 1 KB (codes) and 512 B
// (scales, zeros) so that the tensor-core kernel reads them with full-width,
// conflict-free loads:
//   codes: 32-bit word (gd, kappa, r, c) = gd*64 + kappa*32 + r*4 + c holds, in
//          bytes n = 0..3, the natural byte 8*gd + r of tokens 16*kappa + 4*c + n;
//   scales / zeros: token 16*kappa + 4*c + n sits at row 16*kappa + 4*n + c.
__host__ __device__ __forceinline__ bool value_blocks(int D, int G) { return D == 128 && G == 32; }

// byte offset of natural byte `b` of token `t` (token index inside the layer's
// store) relative to the start of the store of its unit
__host__ __device__ __forceinline__ int64_t vcode_offset(int64_t t, int b, int D, int G) {
    if (!value_blocks(D, G)) return t * (D / 4) + b;
    const int tt = (int)(t & 31);
    const int word = (b >> 3) * 64 + (tt >> 4) * 32 + (b & 7) * 4 + ((tt >> 2) & 3);
    return (t - tt) * 32 + word * 4 + (tt & 3);
}

// index of the (scale, zero) of channel group gd of token t
__host__ __device__ __forceinline__ int64_t vmeta_index(int64_t t, int gd, int D, int G) {
    if (!value_blocks(D, G)) return t * (D / G) + gd;
    const int tt = (int)(t & 31);
    const int row = (tt & 16) | ((tt & 3) << 2) | ((tt >> 2) & 3);
    return ((t - tt) + row) * 4 + gd;
}

__host__ __device__ __forceinline__ int elem_size(int dtype) { return dtype == KIVI_BF16 ? 2 : 4; }

}  // namespace kivi
