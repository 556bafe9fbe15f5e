// Fused decode attention over the packed KIVI cache: tensor-core kernel for
// head_dim 128, group_size 32, up to 8 query heads per KV head in blocks of
// four per CTA (sm_100a).
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
//         its 16-bit half, as the fp16 subnormal c*4^e*2^-24 (one AND per
//         register pair); B = q*s split into fp16 hi + lo parts (the 8 columns
//         are 4 heads x {hi, lo}), 22 significant bits; the zero term is an
//         fp32 dot product per (group, head), computed once per column pair.
//   p.v   out[h,d]   = sum_t (p[h,t]*s[t,gd]) * c[t,d]  +  sum_t p[h,t]*z[t,gd]
//         A = codes of 16 channels x 16 tokens, same encoding; B = p*s in fp16
//         (rounding errors of independent tokens average out), built once per
//         column pair and exchanged by shuffle; the zero term accumulates in fp32.
//   Requires |q*s*sm_scale*log2(e)| and p*s below 65504 (fp16 range).
//
// Data movement: every warp streams its own token groups from HBM into a
// private shared-memory ring with bulk asynchronous copies (cp.async.bulk,
// completion on an mbarrier; six lanes issue one copy each), two groups (8 KB)
// per stage, and unpacks codes in registers.  The unit's queries sit in shared
// memory, pre-scaled.  Nothing dequantized is ever written anywhere.  The
// residual ring (full precision) is handled by extra CTAs with fp32 FMAs.
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
// The packed cache is read once per step: stream it through L2 with an
// evict-first hint (one policy value per thread, made once).
__device__ __forceinline__ uint64_t l2_stream_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// same with a zero addend: starts an accumulator without initialising registers
__device__ __forceinline__ void mma_f16_first(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
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
// A 2-bit code c sitting at bits 2e..2e+1 (e <= 4) of a 16-bit half is, read as
// an fp16 bit pattern with a zero exponent field, the subnormal number
// c * 4^e * 2^-24 -- exactly.  So one AND per register pair turns packed codes
// into a tensor-core operand: no shift, no offset.  The factor 4^e * 2^-24
// belongs to a whole accumulator row and is undone (exactly, a power of two)
// when the accumulator is read.
//
// The tensor core aligns the products of one MMA on their exponent *fields* and
// keeps about 26 bits below the largest (measured: truncation, not rounding).
// A subnormal's field is fixed, so the zero bits above a low-lying code come out
// of that budget: a code at e = 0 is left with 18 bits.  A 32-bit word holds
// four bytes = four codes each; with the bytes of each half swapped (one PRMT,
// in place of the shift that would otherwise bring the odd bytes down) the
// first code of every byte can be taken from bits 8-9 (e = 4) and the other
// three from where they lie (e = 1..3): no row is left with fewer than 20 bits.
template <int E> __device__ __forceinline__ uint32_t code_pair(uint32_t w) {
    static_assert(E >= 0 && E <= 4, "bits 10 and up are the exponent field");
    return w & (0x00030003u << (2 * E));
}
__device__ __forceinline__ uint32_t swap_bytes_in_halves(uint32_t w) { return __byte_perm(w, 0u, 0x2301u); }
constexpr float kRow0 = 65536.0f;             // first code of a byte, taken at e = 4:  2^24 * 4^-4
constexpr float kRow1 = 4194304.0f;           // 2^24 * 4^-1
constexpr float kRow2 = 1048576.0f;           // 2^24 * 4^-2
constexpr float kRow3 = 262144.0f;            // 2^24 * 4^-3

// The eight operand registers of one 32-bit word `w` of codes (bytes b0..b3; the
// halves of a register are MMA k-slots): lo[e] = code e of bytes (b0, b2),
// hi[e] = code e of bytes (b1, b3).
struct CodeRegs { uint32_t lo[4], hi[4]; };
__device__ __forceinline__ CodeRegs code_regs(uint32_t w) {
    const uint32_t ws = swap_bytes_in_halves(w);
    CodeRegs r;
    r.lo[0] = code_pair<4>(ws); r.hi[0] = code_pair<4>(w);
    r.lo[1] = code_pair<1>(w);  r.hi[1] = code_pair<1>(ws);
    r.lo[2] = code_pair<2>(w);  r.hi[2] = code_pair<2>(ws);
    r.lo[3] = code_pair<3>(w);  r.hi[3] = code_pair<3>(ws);
    return r;
}

struct WarpState {
    float m, l;            // running max / sum of head `tig` (score layout)
    float o[8][2];         // p.v sums of 8 channel tiles, rows gid / gid+8 (they still carry 4^I * 2^-24)
    float oz[2];           // zero-point term of head gid>>1, channel groups 2*part and 2*part+1, partial over lanes
};

// ---- one token group (32 tokens) in three phases ----------------------------------
// q.k: scores of the lane's four tokens (4*gid + e) for head `tig`, log2 domain.
// `qx` points at the lane's query slice in shared memory (head hB, pre-scaled,
// channel 4*tig), `qzp`/`kz` at the slice the lane owns for the zero term: the
// hi lane of a column pair takes the even 16-channel steps, the lo lane the odd
// ones, so the dot product q.z is computed once, not twice.
__device__ __forceinline__ void qk_phase(
    const uint8_t* __restrict__ kc, const float* __restrict__ ks, const float* __restrict__ kz,
    const float* __restrict__ qx, const float* __restrict__ qzp, uint32_t part_mask, int gid, int tig, float (&s)[4]) {
    float c0[KIVI_MMA_CHAINS][4], c1[KIVI_MMA_CHAINS][4];
    float qz = 0.0f;
#pragma unroll
    for (int qh = 0; qh < 2; ++qh) {
        const uint4 wv = *reinterpret_cast<const uint4*>(kc + qh * 512 + gid * 64 + tig * 16);
        const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int kt = 4 * qh + m;
            const int ch = 64 * qh + 16 * m;                 // + 4*tig through the lane pointers
            const float4 s4 = *reinterpret_cast<const float4*>(ks + ch);
            const float4 q4 = *reinterpret_cast<const float4*>(qx + ch);
            if ((m & 1) == 0) {                              // channel steps kt, kt+1 -> one of them per lane
                const float4 z4 = *reinterpret_cast<const float4*>(kz + ch);
                const float4 y4 = *reinterpret_cast<const float4*>(qzp + ch);
                qz = fmaf(y4.x, z4.x, qz); qz = fmaf(y4.y, z4.y, qz);
                qz = fmaf(y4.z, z4.z, qz); qz = fmaf(y4.w, z4.w, qz);
            }
            const float x0 = q4.x * s4.x, x1 = q4.y * s4.y, x2 = q4.z * s4.z, x3 = q4.w * s4.w;
            // fp16 hi/lo split of q*s: hi lanes keep x truncated to 11 significant
            // bits, lo lanes keep the remainder (part_mask = 0 on hi lanes)
            const float r0 = x0 - __uint_as_float(__float_as_uint(x0) & part_mask);
            const float r1 = x1 - __uint_as_float(__float_as_uint(x1) & part_mask);
            const float r2 = x2 - __uint_as_float(__float_as_uint(x2) & part_mask);
            const float r3 = x3 - __uint_as_float(__float_as_uint(x3) & part_mask);
            const uint32_t b0 = pack_f16_rz(r0, r2);
            const uint32_t b1 = pack_f16_rz(r1, r3);
            const CodeRegs cr = code_regs(w[m]);
            uint32_t a[4];
            a[0] = cr.lo[0]; a[1] = cr.lo[1]; a[2] = cr.hi[0]; a[3] = cr.hi[1];          // tokens 4*gid, 4*gid + 1
            if (kt < KIVI_MMA_CHAINS) mma_f16_first(c0[kt % KIVI_MMA_CHAINS], a, b0, b1);
            else mma_f16(c0[kt % KIVI_MMA_CHAINS], a, b0, b1);
            a[0] = cr.lo[2]; a[1] = cr.lo[3]; a[2] = cr.hi[2]; a[3] = cr.hi[3];          // tokens 4*gid + 2, + 3
            if (kt < KIVI_MMA_CHAINS) mma_f16_first(c1[kt % KIVI_MMA_CHAINS], a, b0, b1);
            else mma_f16(c1[kt % KIVI_MMA_CHAINS], a, b0, b1);
        }
    }
#pragma unroll
    for (int step = KIVI_MMA_CHAINS / 2; step >= 1; step /= 2)
#pragma unroll
        for (int ch_ = 0; ch_ < step; ++ch_)
#pragma unroll
            for (int i = 0; i < 4; ++i) { c0[ch_][i] += c0[ch_ + step][i]; c1[ch_][i] += c1[ch_ + step][i]; }
    // zero term of head gid>>1: the eight lanes of a column pair hold disjoint partials
    qz += __shfl_xor_sync(0xffffffffu, qz, 1);
    qz += __shfl_xor_sync(0xffffffffu, qz, 2);
    qz += __shfl_xor_sync(0xffffffffu, qz, 4);
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
        for (int mt = 0; mt < 8; ++mt) { st.o[mt][0] *= alpha; st.o[mt][1] *= alpha; }
        const float alpha_b = __shfl_sync(0xffffffffu, alpha, (lane & ~3) | (gid >> 1));
        st.oz[0] *= alpha_b; st.oz[1] *= alpha_b;
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
// 2tig / 2tig+1, bytes 1/3 its k-slots 2tig+8 / 2tig+9 (code_regs).
// The hi and the lo lane of a column pair (gid, gid^1) hold the same head and the
// same tokens, and only the hi lane's B column is ever read.  So the pair splits
// the work by channel group: the hi lane builds p*s and the zero term for groups
// 0,1, the lo lane for groups 2,3, and one exchange hands the hi lane the
// operands it lacks (what the lo lane feeds into its own column is never read).
template <bool FIRST>
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
        // scales / zeros of token 16*kap + 4*tig + n sit at row 16*kap + 4*n + tig;
        // the lane takes the two channel groups 2*part, 2*part + 1 of each row
        float2 sv[4], zv[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            sv[n] = *reinterpret_cast<const float2*>(vs + (16 * kap + 4 * n + tig) * 4 + 2 * part);
            zv[n] = *reinterpret_cast<const float2*>(vz + (16 * kap + 4 * n + tig) * 4 + 2 * part);
        }
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            st.oz[0] = fmaf(pe[n], zv[n].x, st.oz[0]);
            st.oz[1] = fmaf(pe[n], zv[n].y, st.oz[1]);
        }
        uint32_t own[2][2], got[2][2];
        own[0][0] = pack_f16_rn(pe[0] * sv[0].x, pe[2] * sv[2].x);     // k-slots 2tig, 2tig+1: tokens n = 0, 2
        own[0][1] = pack_f16_rn(pe[1] * sv[1].x, pe[3] * sv[3].x);     // k-slots 2tig+8, +9:   tokens n = 1, 3
        own[1][0] = pack_f16_rn(pe[0] * sv[0].y, pe[2] * sv[2].y);
        own[1][1] = pack_f16_rn(pe[1] * sv[1].y, pe[3] * sv[3].y);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j) got[i][j] = __shfl_xor_sync(0xffffffffu, own[i][j], 4);
#pragma unroll
        for (int gd = 0; gd < 4; ++gd) {
            const uint32_t b0 = gd < 2 ? own[gd][0] : got[gd - 2][0];
            const uint32_t b1 = gd < 2 ? own[gd][1] : got[gd - 2][1];
            const CodeRegs cr = code_regs(vw[gd * 64 + kap * 32]);
            uint32_t a[4];
            a[0] = cr.lo[0]; a[1] = cr.lo[1]; a[2] = cr.hi[0]; a[3] = cr.hi[1];          // channels 4*gid, 4*gid + 1 of the group
            if (FIRST && kap == 0) mma_f16_first(acc[2 * gd], a, b0, b1);
            else mma_f16(acc[2 * gd], a, b0, b1);
            a[0] = cr.lo[2]; a[1] = cr.lo[3]; a[2] = cr.hi[2]; a[3] = cr.hi[3];
            if (FIRST && kap == 0) mma_f16_first(acc[2 * gd + 1], a, b0, b1);
            else mma_f16(acc[2 * gd + 1], a, b0, b1);
        }
    }
}

// NG consecutive token groups of one pipeline stage, processed together: the
// q.k and p.v phases of the groups are independent instruction streams, the
// softmax update is done once for all NG*32 tokens.
struct LaneView {
    const float* qx;       // q_s + head*kD + 4*tig
    const float* qzp;      // qx + 16*part
    uint32_t part_mask;    // 0 on hi lanes, "keep 11 significant bits" on lo lanes
    int part, gid, tig, lane;
};

template <int NG>
__device__ __forceinline__ void process_groups(const uint8_t* __restrict__ sb, const LaneView& v, WarpState& st) {
    float s[NG][4];
#pragma unroll
    for (int g = 0; g < NG; ++g)
        qk_phase(sb + g * 1024, reinterpret_cast<const float*>(sb + kGPS * 1024 + g * 512) + 4 * v.tig,
                 reinterpret_cast<const float*>(sb + kGPS * 1536 + g * 512) + 4 * v.tig + 16 * v.part,
                 v.qx, v.qzp, v.part_mask, v.gid, v.tig, s[g]);
    softmax_phase<NG>(s, v.gid, v.lane, st);
    // The tensor core adds each product into its fp32 accumulator with
    // truncation; against an accumulator that has grown over thousands of tokens
    // that is a biased loss (all addends p*s*c are positive) which the later
    // cancellation with the zero term amplifies.  So the MMAs of this stage go
    // into fresh accumulators and join the running sums through ordinary adds
    // (only the even columns are ever read).
    float acc[8][4];
    pv_phase<true>(sb + kGPS * 2048, reinterpret_cast<const float*>(sb + kGPS * 3072),
                   reinterpret_cast<const float*>(sb + kGPS * 3584), s[0], v.part, v.gid, v.tig, acc, st);
#pragma unroll
    for (int g = 1; g < NG; ++g)
        pv_phase<false>(sb + kGPS * 2048 + g * 1024, reinterpret_cast<const float*>(sb + kGPS * 3072 + g * 512),
                        reinterpret_cast<const float*>(sb + kGPS * 3584 + g * 512), s[g], v.part, v.gid, v.tig, acc, st);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) { st.o[mt][0] += acc[mt][0]; st.o[mt][1] += acc[mt][2]; }
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

// grid = units * head blocks * (nq_splits + n_res_splits) CTAs in one dimension
// (head blocks = ceil(n_rep / 4): a CTA serves up to four query heads); block =
// kWarps warps.  The first units*nq_splits CTAs are the quantized pieces, unit by unit:
// piece i of a unit covers token groups [i*gps, min((i+1)*gps, n_groups)).  The
// units*n_res_splits CTAs of the residual ring come last: they are short, so
// the long CTAs start first and the short ones fill the end of the grid
// (measured against ring CTAs first: 3.5 % faster at batch 64 x 32k, 7 % at
// batch 16 x 4k).  Partial slots: quantized piece i -> i, residual part r ->
// nq_splits + r.
//
// Shared memory: [kWarps][kStages][kStageBytes] stage rings | q_s [4][128] fp32
// (the CTA's up to four query heads times sm_scale*log2(e), absent rows zero) | mbarriers |
// (max, sum) of the warps.  When a warp is done, its ring doubles as the
// [4][128] buffer its scaled output goes to; the CTA then adds the warps'
// buffers in warp order (deterministic) and writes one partial.
__global__ void __launch_bounds__(kWarps * 32, KIVI_MMA_MIN_CTAS)
attn_mma_kernel(kivi_layer L, int64_t quant_len, int res_start, int res_len,
                const void* __restrict__ q, int q_dtype,
                float scale_log2, int n_rep, int gps, int nq_splits, int n_res_splits, int res_chunk,
                float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* stage_mem = smem_raw;                                               // [kWarps][kStages][kStageBytes]
    float* q_s = reinterpret_cast<float*>(smem_raw + kWarps * kStages * kStageBytes);   // [4][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_s + 4 * kD);                  // [kWarps][kStages]
    float* ml_s = reinterpret_cast<float*>(bars + kWarps * kStages);             // [kWarps][4][2]

    // the kernel that folds the partials is queued with programmatic stream
    // serialization: let it become resident now, it waits for this grid's end
    cudaTriggerProgrammaticLaunchCompletion();

    // grid order: all quantized pieces (unit-major), then all residual-ring CTAs --
    // the long CTAs start first, the short ones fill the end
    // With more than four query heads per KV head a unit is served by two CTAs per
    // piece, one per block of four heads (they run side by side, so the second
    // read of the piece mostly comes from L2).
    const int head_blocks = (n_rep + 3) >> 2;
    const int n_quant_ctas = (int)L.num_units * head_blocks * nq_splits;
    const bool is_res = (int)blockIdx.x >= n_quant_ctas;
    const int rel = is_res ? (int)blockIdx.x - n_quant_ctas : (int)blockIdx.x;
    const int per_unit = is_res ? n_res_splits : nq_splits;
    const int uv = rel / per_unit, sub = rel - uv * per_unit;
    const int u = uv / head_blocks, head0 = 4 * (uv - u * head_blocks);
    const int n_heads = n_rep - head0 < 4 ? n_rep - head0 : 4;       // heads of this CTA: head0 .. head0 + n_heads - 1
    const int n_splits_total = nq_splits + n_res_splits;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    uint8_t* wstage = stage_mem + warp * kStages * kStageBytes;
    float* fo = reinterpret_cast<float*>(wstage);                               // [4][128] once the ring is idle
    const int slot = is_res ? nq_splits + sub : sub;

    // ---- quantized split: start the copies before anything else ----------------
    const int64_t n_groups = quant_len / kG;
    const int64_t g_begin = is_res ? 0 : (int64_t)slot * gps;
    int64_t g_end = is_res ? 0 : g_begin + gps;
    if (g_end > n_groups) g_end = n_groups;
    const int n_my_groups = (int)(g_end - g_begin);
    const int n_chunks = (n_my_groups + kGPS - 1) / kGPS;
    const int my_n = n_chunks > warp ? (n_chunks - warp + kWarps - 1) / kWarps : 0;
    const uint32_t bar0 = smem_u32(bars + warp * kStages);
    const uint32_t stage0 = smem_u32(wstage);
    // The six pieces of a chunk (key codes, scales, zeros, value codes, scales,
    // zeros) are contiguous runs of 1024 or 512 bytes per token group; lane i < 6
    // owns piece i and issues its copy, so a chunk costs one copy's instructions.
    // Chunk c of this warp starts at group g_begin + (warp + kWarps*c)*kGPS.
    const uint8_t* my_src = nullptr;
    uint32_t my_bytes = 0, my_dst = 0;
    if (!is_res) {
        const uint8_t* base = lane == 0 ? L.k_codes
                            : lane == 1 ? reinterpret_cast<const uint8_t*>(L.k_scales)
                            : lane == 2 ? reinterpret_cast<const uint8_t*>(L.k_zeros)
                            : lane == 3 ? L.v_codes
                            : lane == 4 ? reinterpret_cast<const uint8_t*>(L.v_scales)
                                        : reinterpret_cast<const uint8_t*>(L.v_zeros);
        my_bytes = (lane == 0 || lane == 3) ? 1024u : 512u;
        my_dst = lane == 0 ? 0u : lane == 1 ? kGPS * 1024u : lane == 2 ? kGPS * 1536u
               : lane == 3 ? kGPS * 2048u : lane == 4 ? kGPS * 3072u : kGPS * 3584u;
        const int64_t gw0 = (int64_t)u * (L.max_tokens / kG) + g_begin + (int64_t)warp * kGPS;
        my_src = base + gw0 * my_bytes;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
    }
    const uint64_t policy = l2_stream_policy();
    auto issue = [&](int c) {                 // all lanes call it
        const int goff = (warp + kWarps * c) * kGPS;             // groups from g_begin
        const int ng = (n_my_groups - goff) < kGPS ? (n_my_groups - goff) : kGPS;
        const int s = c % kStages;
        const uint32_t bar = bar0 + 8 * s;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)ng * kGroupBytes);
        __syncwarp();
        if (lane < 6)
            bulk_g2s(stage0 + s * kStageBytes + my_dst, my_src + (int64_t)c * (kWarps * kGPS) * my_bytes,
                     (uint32_t)ng * my_bytes, bar, policy);
    };
    for (int c = 0; c < kStages && c < my_n; ++c) issue(c);

    // ---- queries -> shared memory, pre-scaled -----------------------------------
    {
        for (int i = threadIdx.x; i < kD; i += blockDim.x) {             // 128 float4 = [4][128]
            const int hh = i >> 5, cc = (i & 31) * 4;
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (hh < n_heads) {
                const int64_t e = ((int64_t)u * n_rep + head0 + hh) * kD + cc;
                if (q_dtype == KIVI_BF16) RowVec<__nv_bfloat16>::load4(reinterpret_cast<const __nv_bfloat16*>(q) + e, v);
                else RowVec<float>::load4(reinterpret_cast<const float*>(q) + e, v);
            }
            *reinterpret_cast<float4*>(q_s + hh * kD + cc) =
                make_float4(scale_log2 * v[0], scale_log2 * v[1], scale_log2 * v[2], scale_log2 * v[3]);
        }
    }
    __syncthreads();

    if (is_res) {
        // ---------------- residual ring ----------------
        const int rs = sub;
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
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float M = -INFINITY;
#pragma unroll
            for (int w2 = 0; w2 < kWarps; ++w2) M = fmaxf(M, ml_s[(w2 * 4 + h) * 2]);
            const float f = (m[h] == -INFINITY) ? 0.0f : ex2(m[h] - M);
            *reinterpret_cast<float4*>(fo + h * kD + 4 * lane) = make_float4(f * o[h][0], f * o[h][1], f * o[h][2], f * o[h][3]);
        }
    } else {
        // ---------------- quantized history ----------------
        LaneView v;
        v.part = gid & 1; v.gid = gid; v.tig = tig; v.lane = lane;
        v.qzp = q_s + (gid >> 1) * kD + 4 * tig + 16 * v.part;
        v.qx = q_s + (gid >> 1) * kD + 4 * tig;
        v.part_mask = v.part ? 0xffffe000u : 0u;   // keep 11 significant bits

        WarpState st;
        st.m = -INFINITY; st.l = 0.0f;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) { st.o[mt][0] = 0.0f; st.o[mt][1] = 0.0f; }
        st.oz[0] = 0.0f; st.oz[1] = 0.0f;

        bool ok = true;
        int c = 0;
        for (; c < my_n; ++c) {
            const int s = c % kStages;
            if (!mbar_wait(bar0 + 8 * s, (uint32_t)(c / kStages) & 1u)) { ok = false; break; }
            const int goff = (warp + kWarps * c) * kGPS;
            const uint8_t* sb = wstage + s * kStageBytes;
#if KIVI_MMA_GPS == 2
            if (n_my_groups - goff >= 2) process_groups<2>(sb, v, st);
            else process_groups<1>(sb, v, st);
#else
            process_groups<1>(sb, v, st);
#endif
            __syncwarp();
            if (c + kStages < my_n) issue(c + kStages);
        }
        if (!ok) {
            // A copy did not land within the bound.  The copies still in flight
            // target this warp's ring: give each of them (chunks c .. c+kStages-1,
            // those that were issued) a second bounded wait on its own phase
            // before the ring is reused, then report an empty partial.
            if (lane == 0) atomicExch(&g_fault_word, 1);
            for (int k = c; k < c + kStages && k < my_n; ++k)
                mbar_wait(bar0 + 8 * (k % kStages), (uint32_t)(k / kStages) & 1u);
            st.m = -INFINITY; st.l = 0.0f;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) { st.o[mt][0] = 0.0f; st.o[mt][1] = 0.0f; }
            st.oz[0] = 0.0f; st.oz[1] = 0.0f;
        }

        // ---- fold the warp's lanes ----------------------------------------------
        st.l += __shfl_xor_sync(0xffffffffu, st.l, 4);
        st.l += __shfl_xor_sync(0xffffffffu, st.l, 8);
        st.l += __shfl_xor_sync(0xffffffffu, st.l, 16);
        // zero term: lanes (gid, *) hold head gid>>1, channel groups 2*(gid&1) + {0, 1}
        float ozt[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float z = st.oz[i];
            z += __shfl_xor_sync(0xffffffffu, z, 1);
            z += __shfl_xor_sync(0xffffffffu, z, 2);
            ozt[i] = __shfl_sync(0xffffffffu, z, 8 * tig);          // head tig, group i     <- hi lanes of gid 2*tig
            ozt[2 + i] = __shfl_sync(0xffffffffu, z, 8 * tig + 4);  // head tig, group 2 + i <- lo lanes
        }
        if (gid == 0) { ml_s[(warp * 4 + tig) * 2] = st.m; ml_s[(warp * 4 + tig) * 2 + 1] = st.l; }
        __syncthreads();
        float M = -INFINITY;
#pragma unroll
        for (int w2 = 0; w2 < kWarps; ++w2) M = fmaxf(M, ml_s[(w2 * 4 + tig) * 2]);
        const float f = (st.m == -INFINITY) ? 0.0f : ex2(st.m - M);
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const int gd = mt >> 1;
            const int ch = 32 * gd + 4 * gid + 2 * (mt & 1);
            // rows gid / gid+8 hold code index 2*(mt&1) / 2*(mt&1)+1 of their byte
            const float r0 = (mt & 1) ? kRow2 : kRow0, r1 = (mt & 1) ? kRow3 : kRow1;
            *reinterpret_cast<float2*>(fo + tig * kD + ch) =
                make_float2(f * fmaf(st.o[mt][0], r0, ozt[gd]), f * fmaf(st.o[mt][1], r1, ozt[gd]));
        }
    }
    __syncthreads();

    // ---- the CTA's partial: warps added in warp order ------------------------------
    const int64_t pbase = ((int64_t)u * n_splits_total + slot) * n_rep + head0;
    for (int i = threadIdx.x; i < kD; i += blockDim.x) {
        const int h = i >> 5, cc = (i & 31) * 4;
        if (h < n_heads) {
            float4 a = *reinterpret_cast<const float4*>(stage_mem + h * kD * 4 + cc * 4);
#pragma unroll
            for (int w2 = 1; w2 < kWarps; ++w2) {
                const float4 b = *reinterpret_cast<const float4*>(stage_mem + w2 * kStages * kStageBytes + h * kD * 4 + cc * 4);
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            }
            *reinterpret_cast<float4*>(part_o + (pbase + h) * kD + cc) = a;
        }
    }
    if (threadIdx.x < n_heads) {
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

constexpr size_t kSmemBytes = (size_t)kWarps * kStages * kStageBytes + 4 * kD * 4 + kWarps * kStages * 8 +
                              kWarps * 4 * 2 * 4;
static_assert(kStages * kStageBytes >= 4 * kD * 4, "a warp's ring doubles as its [4][128] fold buffer");
static_assert(kWarps * 32 >= 32, "at least one warp");

}  // namespace

bool attn_mma_supported(const kivi_layer* L, int n_rep, const void* q) {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return L->head_dim == kD && L->group_size == kG && n_rep >= 1 && n_rep <= 8 && al(q) &&
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

// the opt-in shared-memory size is a per-device attribute of the kernel
static int ensure_smem_attr(int* dev_out) {
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    KIVI_CUDA_OK(cudaGetDevice(&dev));
    KIVI_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    if (!attr_set[dev].load(std::memory_order_acquire)) {
        KIVI_CUDA_OK(cudaFuncSetAttribute(attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev].store(true, std::memory_order_release);
    }
    if (dev_out) *dev_out = dev;
    return KIVI_OK;
}

// CTAs of the kernel that one SM holds at a time (registers and shared memory
// decide); asked from the runtime once per device.  0 = the query failed.
int attn_mma_ctas_per_sm() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (ensure_smem_attr(&dev) != KIVI_OK) return 0;
    int n = cached[dev].load(std::memory_order_acquire);
    if (n == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_mma_kernel, kWarps * 32, kSmemBytes) != cudaSuccess || n <= 0)
            return 0;
        cached[dev].store(n, std::memory_order_release);
    }
    return n;
}

int run_attn_mma(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                 const void* q, int q_dtype, int n_rep, float scale_log2, int nq_splits, int gps,
                 int n_res_splits, int res_chunk, float* part_o, float* part_ml, cudaStream_t st) {
    if (int rc = ensure_smem_attr(nullptr)) return rc;
    dim3 grid((unsigned)(nq_splits + n_res_splits) * (unsigned)L->num_units * (unsigned)((n_rep + 3) / 4));
    attn_mma_kernel<<<grid, kWarps * 32, kSmemBytes, st>>>(*L, quant_len, res_start, res_len, q, q_dtype, scale_log2,
                                                         n_rep, gps, nq_splits, n_res_splits, res_chunk, part_o, part_ml);
    KIVI_LAUNCH_OK();
    return KIVI_OK;
}

// ---- self-test: how far below the largest product the tensor core keeps bits -------
// One m16n8k16 MMA per k: C = -1, products {1 * 1, 2^-a * 2^-b} with a + b = k.
// If the unit kept every bit the result would be exactly 2^-k; it aligns the
// addends on their exponent fields and truncates below a fixed distance from the
// largest, so from some k on the small product is lost.  The kernel's accuracy
// budget (code_regs above) assumes at least 24 bits.
__global__ void mma_alignment_probe_kernel(int* kept_out) {
    const int lane = threadIdx.x, gid = lane >> 2, tig = lane & 3;
    int kept = 0;
    for (int k = 8; k <= 34; ++k) {
        const int a_exp = k < 14 ? k : 14, b_exp = k - a_exp;          // both factors stay normal fp16 numbers
        // A[row][0] = 1, A[row][1] = 2^-a; B[0][col] = 1, B[1][col] = 2^-b; everything else 0
        const __half2 a01 = __halves2half2(__float2half(1.0f), __float2half(ldexpf(1.0f, -a_exp)));
        const __half2 b01 = __halves2half2(__float2half(1.0f), __float2half(ldexpf(1.0f, -b_exp)));
        uint32_t a[4] = {0u, 0u, 0u, 0u}, b0 = 0u;
        if (tig == 0) {                                                // k-slots 0 and 1 live in lanes with tig == 0
            a[0] = *reinterpret_cast<const uint32_t*>(&a01);
            a[1] = a[0];
            b0 = *reinterpret_cast<const uint32_t*>(&b01);
        }
        float c[4] = {-1.0f, -1.0f, -1.0f, -1.0f};
        mma_f16(c, a, b0, 0u);
        const bool ok = c[0] == ldexpf(1.0f, -k);
        if (__all_sync(0xffffffffu, ok)) kept = k;
    }
    (void)gid;
    if (lane == 0) *kept_out = kept;
}

int run_mma_alignment_probe(int* bits_out) {
    int* d = nullptr;
    KIVI_CUDA_OK(cudaMalloc(&d, sizeof(int)));
    mma_alignment_probe_kernel<<<1, 32>>>(d);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpy(bits_out, d, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) { set_error("tensor-core alignment probe failed: %s", cudaGetErrorString(e)); return KIVI_ERR_CUDA; }
    return KIVI_OK;
}

int attn_mma_fault_word(int* out) {
    KIVI_CUDA_OK(cudaMemcpyFromSymbol(out, g_fault_word, sizeof(int)));
    return KIVI_OK;
}

int attn_mma_fault_clear() {
    const int zero = 0;
    KIVI_CUDA_OK(cudaMemcpyToSymbol(g_fault_word, &zero, sizeof(int)));
    return KIVI_OK;
}

}  // namespace kivi
