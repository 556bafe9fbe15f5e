// Fused decode attention over the packed KIVI cache: tensor-core kernel for
// head_dim 128, group_size 32, up to 4 query heads per KV head (sm_100a).
//
// Decode attention over 2-bit codes is instruction-bound before it is HBM-bound:
// one quantized (token, kv_head) is 128 bytes of HBM but 256 codes that each
// feed 4 query heads.  The GQA query-group tile therefore runs on the tensor
// cores (mma.sync m16n8k16, fp32 accumulate) with the codes as the exact
// operand, and everything that depends on scales and zeros is folded into the
// small operand:
//
//   q.k   score[t,h] = sum_d (q[h,d]*s[g,d]) * c[d,t]  +  sum_d q[h,d]*z[g,d]
//         A = codes of 16 tokens x 16 channels; a code is used where it lies in
//         its byte, as the fp16 subnormal c*4^e*2^-24 (one AND per register
//         pair, no shift); B = q*s split into fp16 hi + lo parts (the 8 columns
//         are 4 heads x {hi, lo}), 22 significant bits; the zero term is an
//         fp32 dot product per (group, head).
//   p.v   out[h,d]   = sum_t (p[h,t]*s[t,gd]) * c[t,d]  +  sum_t p[h,t]*z[t,gd]
//         A = codes of 16 channels x 16 tokens, same encoding; B = p*s in fp16
//         (rounding errors of independent tokens average out); the zero term
//         accumulates in fp32.
//   Requires |q*s*sm_scale*log2(e)| and p*s below 65504 (fp16 range).
//
// Data movement: every warp streams its own token groups from HBM into a
// private shared-memory ring with bulk asynchronous copies (cp.async.bulk,
// completion on an mbarrier), two groups (8 KB) per stage, and unpacks codes in
// registers.  Nothing dequantized is ever written anywhere.  The residual ring
// (full precision) is one extra split handled with fp32 FMAs.
//
// Every wait on an mbarrier is bounded; on expiry the warp raises the device
// fault word, stops consuming and its partial is written as "empty".
#include "kivi_common.cuh"

#include <cuda_fp16.h>

#include <atomic>

namespace kivi {
namespace {

constexpr int kD = 128, kG = 32;
#ifndef KIVI_MMA_WARPS
#define KIVI_MMA_WARPS 4
#endif
#ifndef KIVI_MMA_GPS
#define KIVI_MMA_GPS 2
#endif
#ifndef KIVI_MMA_STAGES
#define KIVI_MMA_STAGES 2
#endif
#ifndef KIVI_MMA_JOINT
#define KIVI_MMA_JOINT 1            /* 1: both groups of a stage share one softmax update */
#endif
#ifndef KIVI_MMA_CHAINS
#define KIVI_MMA_CHAINS 2           /* independent accumulator chains per q.k tile */
#endif
#ifndef KIVI_MMA_MIN_CTAS
#define KIVI_MMA_MIN_CTAS 3
#endif
constexpr int kWarps = KIVI_MMA_WARPS;     // warps per CTA, each with a private pipeline
constexpr int kGPS = KIVI_MMA_GPS;         // token groups per pipeline stage
constexpr int kStages = KIVI_MMA_STAGES;
constexpr int kGroupBytes = 4096;      // kc 1024 | ks 512 | kz 512 | vc 1024 | vs 512 | vz 512
constexpr int kStageBytes = kGPS * kGroupBytes;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ int g_fault_word = 0;

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false if the barrier did not complete within kSpinLimit polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
#ifndef KIVI_MMA_EVICT_FIRST
#define KIVI_MMA_EVICT_FIRST 1      /* 1: the packed cache is streamed through L2 with an evict-first hint */
#endif
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
#if KIVI_MMA_EVICT_FIRST
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
#else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
#endif
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// {lo16, hi16} = {f16(lo), f16(hi)}
__device__ __forceinline__ uint32_t pack_f16_rz(float lo, float hi) {
    uint32_t r;
    asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16_rn(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


// ---- code -> MMA operand encoding ----------------------------------------------
// A 2-bit code c sitting at bits 2e..2e+1 of the low byte of a 16-bit half is,
// read as an fp16 bit pattern with a zero exponent field, the subnormal number
// c * 4^e * 2^-24 -- exactly.  So one AND per register pair turns packed codes
// into a tensor-core operand: no shift, no offset.  The factor 4^e * 2^-24
// belongs to a whole accumulator row and is undone (exactly, a power of two)
// when the accumulator is read.
template <int E> __device__ __forceinline__ uint32_t code_pair(uint32_t w) {
    return w & (0x00030003u << (2 * E));
}
constexpr float kRow0 = 16777216.0f;          // 2^24 * 4^-0
constexpr float kRow1 = 4194304.0f;           // 2^24 * 4^-1
constexpr float kRow2 = 1048576.0f;           // 2^24 * 4^-2
constexpr float kRow3 = 262144.0f;            // 2^24 * 4^-3

struct WarpState {
    float m, l;            // running max / sum of head `tig` (score layout)
    float o[8][4];         // p.v accumulators, 8 channel tiles (rows still carry 4^I * 2^-24)
    float oz[4];           // zero-point term, head gid>>1, partial over lanes
};

// ---- one token group (32 tokens) in three phases ----------------------------------
// q.k: scores of the lane's four tokens (4*gid + e) for head `tig`, log2 domain.
__device__ __forceinline__ void qk_phase(
    const uint8_t* __restrict__ kc, const float* __restrict__ ks, const float* __restrict__ kz,
    const float* __restrict__ qreg, uint32_t part_mask, int gid, int tig, float (&s)[4]) {
    float c0[KIVI_MMA_CHAINS][4], c1[KIVI_MMA_CHAINS][4];
#pragma unroll
    for (int ch_ = 0; ch_ < KIVI_MMA_CHAINS; ++ch_)
#pragma unroll
        for (int i = 0; i < 4; ++i) { c0[ch_][i] = 0.f; c1[ch_][i] = 0.f; }
    float qz = 0.0f;
#pragma unroll
    for (int qh = 0; qh < 2; ++qh) {
        const uint4 wv = *reinterpret_cast<const uint4*>(kc + qh * 512 + gid * 64 + tig * 16);
        const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int kt = 4 * qh + m;
            const int ch = 64 * qh + 16 * m + 4 * tig;
            const float4 s4 = *reinterpret_cast<const float4*>(ks + ch);
            const float4 z4 = *reinterpret_cast<const float4*>(kz + ch);
            const float4 q4 = *reinterpret_cast<const float4*>(qreg + 4 * kt);
            const float x0 = q4.x * s4.x, x1 = q4.y * s4.y, x2 = q4.z * s4.z, x3 = q4.w * s4.w;
            qz = fmaf(q4.x, z4.x, qz); qz = fmaf(q4.y, z4.y, qz);
            qz = fmaf(q4.z, z4.z, qz); qz = fmaf(q4.w, z4.w, qz);
            // fp16 hi/lo split of q*s: hi lanes keep x truncated to 11 significant
            // bits, lo lanes keep the remainder (part_mask = 0 on hi lanes)
            const float r0 = x0 - __uint_as_float(__float_as_uint(x0) & part_mask);
            const float r1 = x1 - __uint_as_float(__float_as_uint(x1) & part_mask);
            const float r2 = x2 - __uint_as_float(__float_as_uint(x2) & part_mask);
            const float r3 = x3 - __uint_as_float(__float_as_uint(x3) & part_mask);
            const uint32_t b0 = pack_f16_rz(r0, r2);
            const uint32_t b1 = pack_f16_rz(r1, r3);
            const uint32_t we = w[m], wo = w[m] >> 8;
            uint32_t a[4];
            a[0] = code_pair<0>(we); a[1] = code_pair<1>(we); a[2] = code_pair<0>(wo); a[3] = code_pair<1>(wo);
            mma_f16(c0[kt % KIVI_MMA_CHAINS], a, b0, b1);
            a[0] = code_pair<2>(we); a[1] = code_pair<3>(we); a[2] = code_pair<2>(wo); a[3] = code_pair<3>(wo);
            mma_f16(c1[kt % KIVI_MMA_CHAINS], a, b0, b1);
        }
    }
#pragma unroll
    for (int step = KIVI_MMA_CHAINS / 2; step >= 1; step /= 2)
#pragma unroll
        for (int ch_ = 0; ch_ < step; ++ch_)
#pragma unroll
            for (int i = 0; i < 4; ++i) { c0[ch_][i] += c0[ch_ + step][i]; c1[ch_][i] += c1[ch_ + step][i]; }
    // zero term of head gid>>1 (both lanes of a gid pair hold the same partial)
    qz += __shfl_xor_sync(0xffffffffu, qz, 1);
    qz += __shfl_xor_sync(0xffffffffu, qz, 2);
    const float qz_t = __shfl_sync(0xffffffffu, qz, 8 * tig);
    s[0] = fmaf(c0[0][0] + c0[0][1], kRow0, qz_t);   // token 4*gid
    s[1] = fmaf(c0[0][2] + c0[0][3], kRow1, qz_t);   // token 4*gid + 1
    s[2] = fmaf(c1[0][0] + c1[0][1], kRow2, qz_t);   // token 4*gid + 2
    s[3] = fmaf(c1[0][2] + c1[0][3], kRow3, qz_t);   // token 4*gid + 3
}

// running max / sum update for NG groups at once; turns scores into weights
template <int NG>
__device__ __forceinline__ void softmax_phase(float (&s)[NG][4], int gid, int lane, WarpState& st) {
    float gmax = -INFINITY;
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) gmax = fmaxf(gmax, s[g][e]);
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 4));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 8));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 16));
    if (__any_sync(0xffffffffu, gmax > st.m)) {
        const float m_new = fmaxf(st.m, gmax);
        const float alpha = ex2(st.m - m_new);         // 0 when st.m == -inf
        st.m = m_new;
        st.l *= alpha;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) st.o[mt][i] *= alpha;
        const float alpha_b = __shfl_sync(0xffffffffu, alpha, (lane & ~3) | (gid >> 1));
#pragma unroll
        for (int gd = 0; gd < 4; ++gd) st.oz[gd] *= alpha_b;
    }
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) { s[g][e] = ex2(s[g][e] - st.m); st.l += s[g][e]; }
}

// p.v of one group; p[n] = weight of token 4*gid + n for head tig.
// Value block words (kivi_common.cuh): word (gd, kappa, r, c) holds natural byte
// 8*gd + r (channels 32*gd + 4*r + i) of tokens 16*kappa + 4*c + n in bytes n.
// A lane (gid, tig) reads word (gd, kappa, gid, tig): bytes 0/2 are its k-slots
// 2tig / 2tig+1, bytes 1/3 (after >> 8) its k-slots 2tig+8 / 2tig+9.
__device__ __forceinline__ void pv_phase(
    const uint8_t* __restrict__ vc, const float* __restrict__ vs, const float* __restrict__ vz,
    const float (&p)[4], int part, int gid, int tig, float (&acc)[8][4], WarpState& st) {
    const uint32_t* vw = reinterpret_cast<const uint32_t*>(vc) + gid * 4 + tig;
#pragma unroll
    for (int kap = 0; kap < 2; ++kap) {
        const int src = 4 * (4 * kap + tig) + (gid >> 1);   // lane holding tokens 16*kap + 4*tig + n, head gid>>1
        float pe[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) pe[n] = __shfl_sync(0xffffffffu, p[n], src);
        // scales / zeros of token 16*kap + 4*tig + n sit at row 16*kap + 4*n + tig
        float4 sv[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) sv[n] = *reinterpret_cast<const float4*>(vs + (16 * kap + 4 * n + tig) * 4);
        {   // zero term: hi lanes take n = 0,1, lo lanes n = 2,3
            const float pa = part ? pe[2] : pe[0], pb = part ? pe[3] : pe[1];
            const int ra = 16 * kap + 8 * part + tig;
            const float4 za = *reinterpret_cast<const float4*>(vz + ra * 4);
            const float4 zb = *reinterpret_cast<const float4*>(vz + (ra + 4) * 4);
            st.oz[0] = fmaf(pa, za.x, fmaf(pb, zb.x, st.oz[0]));
            st.oz[1] = fmaf(pa, za.y, fmaf(pb, zb.y, st.oz[1]));
            st.oz[2] = fmaf(pa, za.z, fmaf(pb, zb.z, st.oz[2]));
            st.oz[3] = fmaf(pa, za.w, fmaf(pb, zb.w, st.oz[3]));
        }
        // lo lanes feed the odd B columns with the same p*s: those columns of the
        // accumulators are never read
#pragma unroll
        for (int gd = 0; gd < 4; ++gd) {
            const float s0 = gd == 0 ? sv[0].x : gd == 1 ? sv[0].y : gd == 2 ? sv[0].z : sv[0].w;
            const float s1 = gd == 0 ? sv[1].x : gd == 1 ? sv[1].y : gd == 2 ? sv[1].z : sv[1].w;
            const float s2 = gd == 0 ? sv[2].x : gd == 1 ? sv[2].y : gd == 2 ? sv[2].z : sv[2].w;
            const float s3 = gd == 0 ? sv[3].x : gd == 1 ? sv[3].y : gd == 2 ? sv[3].z : sv[3].w;
            const uint32_t b0 = pack_f16_rn(pe[0] * s0, pe[2] * s2);     // k-slots 2tig, 2tig+1: tokens n = 0, 2
            const uint32_t b1 = pack_f16_rn(pe[1] * s1, pe[3] * s3);     // k-slots 2tig+8, +9:   tokens n = 1, 3
            const uint32_t we = vw[gd * 64 + kap * 32], wo = we >> 8;
            uint32_t a[4];
            a[0] = code_pair<0>(we); a[1] = code_pair<1>(we); a[2] = code_pair<0>(wo); a[3] = code_pair<1>(wo);
            mma_f16(acc[2 * gd], a, b0, b1);
            a[0] = code_pair<2>(we); a[1] = code_pair<3>(we); a[2] = code_pair<2>(wo); a[3] = code_pair<3>(wo);
            mma_f16(acc[2 * gd + 1], a, b0, b1);
        }
    }
}

// NG consecutive token groups of one pipeline stage, processed together: the
// q.k and p.v phases of the groups are independent instruction streams, the
// softmax update is done once for all NG*32 tokens.
template <int NG>
__device__ __forceinline__ void process_groups(
    const uint8_t* __restrict__ sb, int g0, const float* __restrict__ qreg, uint32_t part_mask,
    int part, int gid, int tig, int lane, WarpState& st) {
    float s[NG][4];
#pragma unroll
    for (int g = 0; g < NG; ++g)
        qk_phase(sb + (g0 + g) * 1024, reinterpret_cast<const float*>(sb + kGPS * 1024 + (g0 + g) * 512),
                 reinterpret_cast<const float*>(sb + kGPS * 1536 + (g0 + g) * 512), qreg, part_mask, gid, tig, s[g]);
    softmax_phase<NG>(s, gid, lane, st);
    // The tensor core adds each product into its fp32 accumulator with
    // truncation; against an accumulator that has grown over thousands of tokens
    // that is a biased loss (all addends p*s*c are positive) which the later
    // cancellation with the zero term amplifies.  So the MMAs of this stage go
    // into fresh accumulators and join the running sums through ordinary adds
    // (only the even columns are ever read).
    float acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
#pragma unroll
    for (int g = 0; g < NG; ++g)
        pv_phase(sb + kGPS * 2048 + (g0 + g) * 1024, reinterpret_cast<const float*>(sb + kGPS * 3072 + (g0 + g) * 512),
                 reinterpret_cast<const float*>(sb + kGPS * 3584 + (g0 + g) * 512), s[g], part, gid, tig, acc, st);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) { st.o[mt][0] += acc[mt][0]; st.o[mt][2] += acc[mt][2]; }
}

// ---- residual ring: full-precision tokens ---------------------------------------
// CTA `rs` of the residual part handles window tokens [rs*chunk, (rs+1)*chunk).
// A warp takes 32 tokens at a time: lane = (4 tokens, quarter of the channels)
// for q.k (vector loads of 32 channels, 2 shuffles to finish the dot products),
// then lane = 4 channels for p.v.  Result: per warp (m, l, o) for 4 heads, merged
// through shared memory like the quantized splits.
template <typename T> struct RowVec;
template <> struct RowVec<float> {
    __device__ static void load8(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    __device__ static void load4(const float* p, float (&v)[4]) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
};
template <> struct RowVec<__nv_bfloat16> {
    __device__ static void load8(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
    __device__ static void load4(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
        v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
    }
};

template <typename T>
__device__ __forceinline__ void residual_part(
    const T* __restrict__ k_res, const T* __restrict__ v_res, int R, int res_start, int res_len,
    int t_begin, int t_end, const float* __restrict__ q_s /* [4][128], pre-scaled */,
    int lane, int warp, float (&m)[4], float (&l)[4], float (&o)[4][4]) {
    const int tl = lane >> 2, cq = lane & 3;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) o[h][i] = 0.0f;
    }
    // a warp pass covers 32 tokens: lane (tl, cq) holds tokens t0 + tl + 8j, j = 0..3,
    // and channels 32*cq .. 32*cq+31 of each; every q vector read feeds 4 tokens
    for (int t0 = t_begin + 32 * warp; t0 < t_end; t0 += 32 * kWarps) {
        float acc[4][4];
        const T* row[4];
        bool valid[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = t0 + tl + 8 * j;
            valid[j] = t < t_end;
            int slot = res_start + (valid[j] ? t : t0);              // both below R
            if (slot >= R) slot -= R;
            row[j] = k_res + (int64_t)slot * kD + 32 * cq;
#pragma unroll
            for (int h = 0; h < 4; ++h) acc[j][h] = 0.0f;
        }
#pragma unroll 2
        for (int c = 0; c < 4; ++c) {
            float kv[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j) RowVec<T>::load8(row[j] + 8 * c, kv[j]);
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const float4 qa = *reinterpret_cast<const float4*>(q_s + h * kD + 32 * cq + 8 * c);
                const float4 qb = *reinterpret_cast<const float4*>(q_s + h * kD + 32 * cq + 8 * c + 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a = acc[j][h];
                    a = fmaf(kv[j][0], qa.x, a); a = fmaf(kv[j][1], qa.y, a);
                    a = fmaf(kv[j][2], qa.z, a); a = fmaf(kv[j][3], qa.w, a);
                    a = fmaf(kv[j][4], qb.x, a); a = fmaf(kv[j][5], qb.y, a);
                    a = fmaf(kv[j][6], qb.z, a); a = fmaf(kv[j][7], qb.w, a);
                    acc[j][h] = a;
                }
            }
        }
        float p[4][4];     // [j][h]
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float sc = acc[j][h];
                sc += __shfl_xor_sync(0xffffffffu, sc, 1);
                sc += __shfl_xor_sync(0xffffffffu, sc, 2);
                acc[j][h] = valid[j] ? sc : -INFINITY;
                mx = fmaxf(mx, acc[j][h]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m[h], mx);          // finite: token t0 is always valid
            const float alpha = ex2(m[h] - m_new);
            m[h] = m_new;
            float ps = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) { p[j][h] = valid[j] ? ex2(acc[j][h] - m_new) : 0.0f; ps += p[j][h]; }
            // the four lanes of a token quad hold the same p: count it once
            l[h] = l[h] * alpha + (cq == 0 ? ps : 0.0f);
#pragma unroll
            for (int i = 0; i < 4; ++i) o[h][i] *= alpha;
        }
        const int ntok = t_end - t0 < 32 ? t_end - t0 : 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (8 * j >= ntok) break;
            // eight value rows in flight at once; a token past the end re-reads
            // row t0 and carries p = 0
            float vv[8][4];
#pragma unroll
            for (int tk = 0; tk < 8; ++tk) {
                int slot = res_start + t0 + (8 * j + tk < ntok ? 8 * j + tk : 0);
                if (slot >= R) slot -= R;
                RowVec<T>::load4(v_res + (int64_t)slot * kD + 4 * lane, vv[tk]);
            }
#pragma unroll
            for (int tk = 0; tk < 8; ++tk) {
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float ph = __shfl_sync(0xffffffffu, p[j][h], 4 * tk);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[h][i] = fmaf(ph, vv[tk][i], o[h][i]);
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 4; ++h) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], off);
    }
}

// grid = (n_res_splits + nq_splits, units); block = kWarps warps.  The first
// n_res_splits CTAs of a unit take the residual ring (they are scheduled first
// and overlap with the rest); CTA n_res_splits + i covers token groups
// [i*gps, min((i+1)*gps, n_groups)).  Partial slots: quantized split i -> i,
// residual part r -> nq_splits + r.
__global__ void __launch_bounds__(kWarps * 32, KIVI_MMA_MIN_CTAS)
attn_mma_kernel(kivi_layer L, int64_t quant_len, int res_start, int res_len,
                const void* __restrict__ q, int q_dtype,
                float scale_log2, int n_rep, int gps, int nq_splits, int n_res_splits, int res_chunk,
                float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* stage_mem = smem_raw;                                               // [kWarps][kStages][kStageBytes]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kWarps * kStages * kStageBytes);  // [kWarps][kStages]
    float* ml_s = reinterpret_cast<float*>(bars + kWarps * kStages);             // [kWarps][4][2]
    float* o_s = ml_s + kWarps * 4 * 2;                                          // [4][128]

    const int u = blockIdx.y;
    const int n_splits_total = nq_splits + n_res_splits;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;

    if ((int)blockIdx.x < n_res_splits) {
        // ---------------- residual ring ----------------
        const int rs = blockIdx.x;
        float* q_s = reinterpret_cast<float*>(stage_mem);            // [4][128]
        for (int i = threadIdx.x; i < 4 * kD; i += blockDim.x) {
            const int h = i / kD;
            q_s[i] = h < n_rep ? scale_log2 * load_as_float(q, q_dtype, (int64_t)u * n_rep * kD + i) : 0.0f;
        }
        for (int i = threadIdx.x; i < 4 * kD; i += blockDim.x) o_s[i] = 0.0f;
        __syncthreads();
        const int t_begin = rs * res_chunk;
        const int t_end = t_begin + res_chunk < res_len ? t_begin + res_chunk : res_len;
        float m[4], l[4], o[4][4];
        if (L.res_dtype == KIVI_BF16)
            residual_part<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(L.k_res) + (int64_t)u * L.residual_cap * kD,
                                         reinterpret_cast<const __nv_bfloat16*>(L.v_res) + (int64_t)u * L.residual_cap * kD,
                                         L.residual_cap, res_start, res_len, t_begin, t_end, q_s, lane, warp, m, l, o);
        else
            residual_part<float>(reinterpret_cast<const float*>(L.k_res) + (int64_t)u * L.residual_cap * kD,
                                 reinterpret_cast<const float*>(L.v_res) + (int64_t)u * L.residual_cap * kD,
                                 L.residual_cap, res_start, res_len, t_begin, t_end, q_s, lane, warp, m, l, o);
        if (lane < 4) {
            // lane h publishes head h (m and l are warp-uniform after the reductions)
            float mh = m[0], lh = l[0];
            if (lane == 1) { mh = m[1]; lh = l[1]; }
            if (lane == 2) { mh = m[2]; lh = l[2]; }
            if (lane == 3) { mh = m[3]; lh = l[3]; }
            ml_s[(warp * 4 + lane) * 2] = mh; ml_s[(warp * 4 + lane) * 2 + 1] = lh;
        }
        __syncthreads();
        for (int w2 = 0; w2 < kWarps; ++w2) {
            if (warp == w2) {
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    float M = -INFINITY;
                    for (int w3 = 0; w3 < kWarps; ++w3) M = fmaxf(M, ml_s[(w3 * 4 + h) * 2]);
                    const float f = (m[h] == -INFINITY) ? 0.0f : ex2(m[h] - M);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o_s[h * kD + 4 * lane + i] += f * o[h][i];
                }
            }
            __syncthreads();
        }
        const int64_t pbase = ((int64_t)u * n_splits_total + nq_splits + rs) * n_rep;
        for (int i = threadIdx.x; i < n_rep * kD; i += blockDim.x) part_o[pbase * kD + i] = o_s[i];
        if (threadIdx.x < n_rep) {
            const int h = threadIdx.x;
            float Mh = -INFINITY, ls = 0.0f;
            for (int w2 = 0; w2 < kWarps; ++w2) Mh = fmaxf(Mh, ml_s[(w2 * 4 + h) * 2]);
            for (int w2 = 0; w2 < kWarps; ++w2) {
                const float mw = ml_s[(w2 * 4 + h) * 2];
                if (mw != -INFINITY) ls += ml_s[(w2 * 4 + h) * 2 + 1] * ex2(mw - Mh);
            }
            part_ml[(pbase + h) * 2] = Mh;
            part_ml[(pbase + h) * 2 + 1] = ls;
        }
        return;
    }
    const int split = (int)blockIdx.x - n_res_splits;
    const int part = gid & 1, hB = gid >> 1;
    const int64_t max_groups = L.max_tokens / kG;
    const int64_t n_groups = quant_len / kG;
    const int64_t g_begin = (int64_t)split * gps;
    int64_t g_end = g_begin + gps;
    if (g_end > n_groups) g_end = n_groups;
    const int n_chunks = (int)((g_end - g_begin + kGPS - 1) / kGPS);
    const int my_n = n_chunks > warp ? (n_chunks - warp + kWarps - 1) / kWarps : 0;

    uint8_t* wstage = stage_mem + warp * kStages * kStageBytes;
    const uint32_t bar0 = smem_u32(bars + warp * kStages);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // chunk i of this warp starts at group g_begin + (warp + kWarps*i)*kGPS: base
    // pointers of chunk 0, advanced by a constant per chunk
    const int64_t gw0 = (int64_t)u * max_groups + g_begin + (int64_t)warp * kGPS;
    const int64_t tw0 = (int64_t)u * L.max_tokens + (g_begin + (int64_t)warp * kGPS) * kG;
    const uint8_t* pk_c = L.k_codes + gw0 * 1024;
    const float* pk_s = L.k_scales + gw0 * kD;
    const float* pk_z = L.k_zeros + gw0 * kD;
    const uint8_t* pv_c = L.v_codes + tw0 * 32;
    const float* pv_s = L.v_scales + tw0 * 4;
    const float* pv_z = L.v_zeros + tw0 * 4;
    const int n_my_groups = (int)(g_end - g_begin);
    auto issue = [&](int i) {
        const int goff = (warp + kWarps * i) * kGPS;             // groups from g_begin
        const int ng = (n_my_groups - goff) < kGPS ? (n_my_groups - goff) : kGPS;
        const int s = i % kStages;
        const uint32_t bar = bar0 + 8 * s;
        const uint32_t dst = smem_u32(wstage + s * kStageBytes);
        const int64_t adv = (int64_t)i * kWarps * kGPS;          // groups past chunk 0
        mbar_expect_tx(bar, (uint32_t)ng * kGroupBytes);
        bulk_g2s(dst, pk_c + adv * 1024, ng * 1024, bar);
        bulk_g2s(dst + kGPS * 1024, pk_s + adv * kD, ng * 512, bar);
        bulk_g2s(dst + kGPS * 1536, pk_z + adv * kD, ng * 512, bar);
        bulk_g2s(dst + kGPS * 2048, pv_c + adv * 1024, ng * 1024, bar);
        bulk_g2s(dst + kGPS * 3072, pv_s + adv * 128, ng * 512, bar);
        bulk_g2s(dst + kGPS * 3584, pv_z + adv * 128, ng * 512, bar);
    };
    if (lane == 0) {
        for (int i = 0; i < kStages && i < my_n; ++i) issue(i);
    }

    // query registers: channel 64*qh + 16*m + 4*tig + i at index 16*qh + 4*m + i,
    // head hB, pre-multiplied by sm_scale * log2(e)
    __align__(16) float qreg[32];
    {
        const float f = scale_log2;
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            const int ch = 64 * (r >> 4) + 16 * ((r >> 2) & 3) + 4 * tig + (r & 3);
            qreg[r] = hB < n_rep ? f * load_as_float(q, q_dtype, ((int64_t)u * n_rep + hB) * kD + ch) : 0.0f;
        }
    }
    const uint32_t part_mask = part ? 0xffffe000u : 0u;   // keep 11 significant bits

    WarpState st;
    st.m = -INFINITY; st.l = 0.0f;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) st.o[mt][i] = 0.0f;
#pragma unroll
    for (int gd = 0; gd < 4; ++gd) {
        st.oz[gd] = 0.0f;
    }

    bool ok = true;
    for (int i = 0; i < my_n; ++i) {
        const int s = i % kStages;
        if (!mbar_wait(bar0 + 8 * s, (uint32_t)(i / kStages) & 1u)) { ok = false; break; }
        const int64_t g0 = g_begin + (int64_t)(warp + kWarps * i) * kGPS;
        const int ng = (int)((g_end - g0) < kGPS ? (g_end - g0) : kGPS);
        const uint8_t* sb = wstage + s * kStageBytes;
#if KIVI_MMA_JOINT
        static_assert(kGPS == 2, "joint processing is written for two groups per stage");
        if (ng == 2) {
            process_groups<2>(sb, 0, qreg, part_mask, part, gid, tig, lane, st);
        } else {
            process_groups<1>(sb, 0, qreg, part_mask, part, gid, tig, lane, st);
        }
#else
        for (int gi = 0; gi < ng; ++gi)
            process_groups<1>(sb, gi, qreg, part_mask, part, gid, tig, lane, st);
#endif
        __syncwarp();
        if (lane == 0 && i + kStages < my_n) issue(i + kStages);
    }
    if (!ok) {
        // copies still in flight target this CTA's shared memory: give them a
        // bounded chance to land before the CTA may exit, then report empty.
        if (lane == 0) atomicExch(&g_fault_word, 1);
        for (int s = 0; s < kStages; ++s) mbar_wait(bar0 + 8 * s, 0);
        st.m = -INFINITY; st.l = 0.0f;
    }

    // ---- fold the warp's lanes, then the CTA's warps ---------------------------
    st.l += __shfl_xor_sync(0xffffffffu, st.l, 4);
    st.l += __shfl_xor_sync(0xffffffffu, st.l, 8);
    st.l += __shfl_xor_sync(0xffffffffu, st.l, 16);
    float ozt[4];
#pragma unroll
    for (int gd = 0; gd < 4; ++gd) {
        float z = st.oz[gd];
        z += __shfl_xor_sync(0xffffffffu, z, 1);
        z += __shfl_xor_sync(0xffffffffu, z, 2);
        z += __shfl_xor_sync(0xffffffffu, z, 4);      // the other half of the tokens (lo lanes)
        ozt[gd] = __shfl_sync(0xffffffffu, z, 8 * tig);   // head tig <- lanes with gid>>1 == tig
    }
    if (gid == 0) { ml_s[(warp * 4 + tig) * 2] = st.m; ml_s[(warp * 4 + tig) * 2 + 1] = st.l; }
    for (int i = threadIdx.x; i < 4 * kD; i += blockDim.x) o_s[i] = 0.0f;
    __syncthreads();
    float M = -INFINITY;
    for (int w2 = 0; w2 < kWarps; ++w2) M = fmaxf(M, ml_s[(w2 * 4 + tig) * 2]);
    const float f = (st.m == -INFINITY) ? 0.0f : ex2(st.m - M);
    for (int w2 = 0; w2 < kWarps; ++w2) {
        if (warp == w2 && f != 0.0f) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const int gd = mt >> 1;
                const int ch = 32 * gd + 4 * gid + 2 * (mt & 1);
                // rows gid / gid+8 hold code index 2*(mt&1) / 2*(mt&1)+1 of their byte
                const float r0 = (mt & 1) ? kRow2 : kRow0, r1 = (mt & 1) ? kRow3 : kRow1;
                o_s[tig * kD + ch] += f * fmaf(st.o[mt][0], r0, ozt[gd]);       // odd columns unused
                o_s[tig * kD + ch + 1] += f * fmaf(st.o[mt][2], r1, ozt[gd]);
            }
        }
        __syncthreads();
    }
    const int64_t pbase = ((int64_t)u * n_splits_total + split) * n_rep;
    for (int i = threadIdx.x; i < n_rep * kD; i += blockDim.x)
        part_o[pbase * kD + i] = o_s[i];
    if (threadIdx.x < n_rep) {
        const int h = threadIdx.x;
        float Mh = -INFINITY, ls = 0.0f;
        for (int w2 = 0; w2 < kWarps; ++w2) Mh = fmaxf(Mh, ml_s[(w2 * 4 + h) * 2]);
        for (int w2 = 0; w2 < kWarps; ++w2) {
            const float mw = ml_s[(w2 * 4 + h) * 2];
            if (mw != -INFINITY) ls += ml_s[(w2 * 4 + h) * 2 + 1] * ex2(mw - Mh);
        }
        part_ml[(pbase + h) * 2] = Mh;
        part_ml[(pbase + h) * 2 + 1] = ls;
    }
}

constexpr size_t kSmemBytes = (size_t)kWarps * kStages * kStageBytes + kWarps * kStages * 8 +
                              kWarps * 4 * 2 * 4 + 4 * kD * 4;

}  // namespace

bool attn_mma_supported(const kivi_layer* L, int n_rep, int q_dtype) {
    (void)q_dtype;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return L->head_dim == kD && L->group_size == kG && n_rep >= 1 && n_rep <= 4 &&
           al(L->k_res) && al(L->v_res) && al(L->k_codes) && al(L->k_scales) && al(L->k_zeros) && al(L->v_codes) && al(L->v_scales) && al(L->v_zeros);
}

// number of residual CTAs per unit and tokens per CTA (multiple of 32)
void attn_mma_residual_plan(int res_len, int* n_res_splits, int* res_chunk) {
    int rs = (res_len + 32 * kWarps - 1) / (32 * kWarps);
    if (rs > 8) rs = 8;
    int chunk = rs ? (res_len + rs - 1) / rs : 0;
    chunk = (chunk + 31) / 32 * 32;
    *n_res_splits = chunk ? (res_len + chunk - 1) / chunk : 0;
    *res_chunk = chunk;
}

int run_attn_mma(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                 const void* q, int q_dtype, int n_rep, float scale_log2, int nq_splits, int gps,
                 int n_res_splits, int res_chunk, float* part_o, float* part_ml, cudaStream_t st) {
    // the opt-in shared-memory size is a per-device attribute of the kernel
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    KIVI_CUDA_OK(cudaGetDevice(&dev));
    KIVI_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        KIVI_CUDA_OK(cudaFuncSetAttribute(attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev].store(true, std::memory_order_release);
    }
    dim3 grid((unsigned)(nq_splits + n_res_splits), (unsigned)L->num_units);
    attn_mma_kernel<<<grid, kWarps * 32, kSmemBytes, st>>>(*L, quant_len, res_start, res_len, q, q_dtype, scale_log2,
                                                         n_rep, gps, nq_splits, n_res_splits, res_chunk, part_o, part_ml);
    KIVI_LAUNCH_OK();
    return KIVI_OK;
}

int attn_mma_fault_word(int* out) {
    KIVI_CUDA_OK(cudaMemcpyFromSymbol(out, g_fault_word, sizeof(int)));
    return KIVI_OK;
}

}  // namespace kivi
