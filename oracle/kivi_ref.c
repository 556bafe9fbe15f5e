/* Plain-C restatement of the reference's device arithmetic.
 * TEST INFRASTRUCTURE ONLY: only tests/, the smoke check and the CPU-baseline
 * leg of the benchmark may load the library built from this file.
 *
 * Follows the reference's kernel sources (half-away rounding, NaN-ignoring
 * min/max starting at +-1e30f), not its torch mirror:
 *   min/max   src/csrc/kernels/internal/quant_tile.hpp:35-49
 *   pack      src/csrc/kernels/internal/quant_tile.hpp:53-70
 *   roundtrip src/csrc/kernels/internal/quant_tile.hpp:74-91
 *   scale     src/csrc/kernels/quantize_kernels.cpp:46-48
 *   dequant   src/csrc/kernels/dequantize_kernels.cpp:17-28, 50-61
 * Build with -O2 -ffp-contract=off (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>

static void group_min_max(const float* x, int n, float* mn, float* mx) {
    float lo = 1e30f, hi = -1e30f;
    for (int i = 0; i < n; ++i) {
        lo = fminf(lo, x[i]);
        hi = fmaxf(hi, x[i]);
    }
    *mn = lo;
    *mx = hi;
}

static int code_of(float v, float mn, float scale, int half_even) {
    float t = (v - mn) / scale;
    int q = (int)(half_even ? rintf(t) : roundf(t));
    return q < 0 ? 0 : (q > 3 ? 3 : q);
}

void kivi_c_quantize_groups(const float* in, uint8_t* packed, float* scales,
                            float* zeros, long num_groups, int group_size,
                            int half_even) {
    for (long g = 0; g < num_groups; ++g) {
        const float* x = in + g * (long)group_size;
        float mn, mx;
        group_min_max(x, group_size, &mn, &mx);
        float scale = (mx - mn) / 3.0f + 1e-10f;
        scales[g] = scale;
        zeros[g] = mn;
        for (int i = 0; i < group_size; i += 4) {
            unsigned b = 0;
            for (int j = 0; j < 4; ++j)
                b |= (unsigned)code_of(x[i + j], mn, scale, half_even) << (2 * j);
            packed[g * (long)(group_size / 4) + i / 4] = (uint8_t)b;
        }
    }
}

void kivi_c_dequantize_groups(const uint8_t* packed, const float* scales,
                              const float* zeros, float* out, long num_groups,
                              int group_size) {
    long bytes_per_group = group_size / 4;
    for (long g = 0; g < num_groups; ++g) {
        float s = scales[g], z = zeros[g];
        for (long b = 0; b < bytes_per_group; ++b) {
            unsigned p = packed[g * bytes_per_group + b];
            for (int j = 0; j < 4; ++j) {
                float prod = (float)((p >> (2 * j)) & 3u) * s;
                out[g * (long)group_size + b * 4 + j] = prod + z;
            }
        }
    }
}

void kivi_c_roundtrip_groups(const float* in, float* out, long num_groups,
                             int group_size, int half_even) {
    for (long g = 0; g < num_groups; ++g) {
        const float* x = in + g * (long)group_size;
        float mn, mx;
        group_min_max(x, group_size, &mn, &mx);
        float scale = (mx - mn) / 3.0f + 1e-10f;
        for (int i = 0; i < group_size; ++i) {
            float prod = (float)code_of(x[i], mn, scale, half_even) * scale;
            out[g * (long)group_size + i] = prod + mn;
        }
    }
}
