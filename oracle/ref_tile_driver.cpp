// CPU driver around the reference's own per-group device helpers.
// TEST INFRASTRUCTURE ONLY.
//
// Compiles the reference header src/csrc/kernels/internal/quant_tile.hpp where
// it lies (found through -I, never copied) against oracle/sycl_shim, and walks
// the groups the way the reference's launch bodies do:
//   quantize : src/csrc/kernels/quantize_kernels.cpp:39-51 (one work-item per
//              group: reduce -> scale/zero -> pack)
//   roundtrip: src/csrc/kernels/roundtrip_kernels.cpp:27-33
// The values-per-token kernels (quantize_kernels.cpp:88-103,
// roundtrip_kernels.cpp:64-75) address the same flat runs of group_size
// elements (base == gid*group_size because groups_per_token*group_size ==
// head_dim), so one flat walk covers both.
//
// Built with -O2 -ffp-contract=off so "q*scale + min" stays a separate multiply
// and add.  The output goes to oracle/_ref/ only.
#include <cstdint>
#include "kernels/internal/quant_tile.hpp"

extern "C" {

void ref_quantize_groups(const float* in, uint8_t* packed, float* scales,
                         float* zeros, long num_groups, int group_size) {
    for (long g = 0; g < num_groups; ++g) {
        // the reference indexes with int; the checker is only run on inputs
        // below 2^31 elements, in blocks re-based per call
        const float* base_ptr = in + g * group_size;
        float mn, mx;
        kivi::detail::reduce_min_max_vec(base_ptr, 0, group_size, mn, mx);
        float scale = (mx - mn) / 3.0f + 1e-10f;
        scales[g] = scale;
        zeros[g] = mn;
        kivi::detail::pack_vec(base_ptr, 0, group_size, mn, scale,
                               packed + g * (group_size / 4), 0);
    }
}

void ref_roundtrip_groups(const float* in, float* out, long num_groups,
                          int group_size) {
    for (long g = 0; g < num_groups; ++g) {
        const float* base_ptr = in + g * group_size;
        float mn, mx;
        kivi::detail::reduce_min_max_vec(base_ptr, 0, group_size, mn, mx);
        float scale = (mx - mn) / 3.0f + 1e-10f;
        kivi::detail::roundtrip_vec(base_ptr, 0, group_size, mn, scale,
                                    out + g * group_size, 0);
    }
}

}  // extern "C"
