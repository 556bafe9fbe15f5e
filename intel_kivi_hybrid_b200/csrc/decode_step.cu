// One decode layer-step fed from and returning to pinned host memory:
//   host q + the step's new K/V token -> ring append (+ flush on one step in G)
//   -> fused attention -> outputs in host memory,
// as ONE call of the C ABI, so a host loop pays one foreign call per step instead
// of five.  Two ways to move the data (about 1.3 MB per step at batch 64):
//   direct  the kernels read q and the new token from, and write the outputs to,
//           the pinned host buffers themselves (pinned memory is addressable from
//           the device): no copy operations at all, the bytes cross PCIe while
//           the kernels run;
//   staged  explicit copies into a device staging buffer and back, with the units
//           optionally cut into chunks on separate streams so that one chunk's
//           copies overlap another's kernels.
//
// What it replaces in the reference: the body of one generate() iteration around
// the model forward -- get_full_cache() + add_tokens() (generation/generate.py:
// 72-77, cache/manager.py:162-290), there a host-side cat/flush/serve per step.
#include <mutex>

#include "kivi_common.cuh"

namespace kivi {
namespace {

constexpr int kMaxChunks = 4;
constexpr int kMaxDevices = 64;

struct SideStreams {
    bool ready = false;
    cudaStream_t side[kMaxChunks - 1];
    cudaEvent_t fork, join[kMaxChunks - 1];
};
SideStreams g_side[kMaxDevices];
std::mutex g_side_mutex;

int side_streams(SideStreams** out) {
    int dev = 0;
    KIVI_CUDA_OK(cudaGetDevice(&dev));
    KIVI_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d outside 0..%d", dev, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_side_mutex);
    SideStreams& s = g_side[dev];
    if (!s.ready) {
        for (int i = 0; i < kMaxChunks - 1; ++i) {
            KIVI_CUDA_OK(cudaStreamCreateWithFlags(&s.side[i], cudaStreamNonBlocking));
            KIVI_CUDA_OK(cudaEventCreateWithFlags(&s.join[i], cudaEventDisableTiming));
        }
        KIVI_CUDA_OK(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
        s.ready = true;
    }
    *out = &s;
    return KIVI_OK;
}

// `layer` restricted to units [u0, u1)
kivi_layer slice_units(const kivi_layer* L, int u0, int u1) {
    kivi_layer s = *L;
    const int64_t D = L->head_dim, G = L->group_size, mt = L->max_tokens, mg = mt / G, R = L->residual_cap;
    const int64_t esz = elem_size(L->res_dtype);
    s.num_units = u1 - u0;
    s.k_codes = L->k_codes + (int64_t)u0 * mg * (D * G / 4);
    s.k_scales = L->k_scales + (int64_t)u0 * mg * D;
    s.k_zeros = L->k_zeros + (int64_t)u0 * mg * D;
    s.v_codes = L->v_codes + (int64_t)u0 * mt * (D / 4);
    s.v_scales = L->v_scales + (int64_t)u0 * mt * (D / G);
    s.v_zeros = L->v_zeros + (int64_t)u0 * mt * (D / G);
    s.k_res = reinterpret_cast<uint8_t*>(L->k_res) + (int64_t)u0 * R * D * esz;
    s.v_res = reinterpret_cast<uint8_t*>(L->v_res) + (int64_t)u0 * R * D * esz;
    return s;
}

}  // namespace
}  // namespace kivi

using namespace kivi;

extern "C" size_t kivi_decode_step_stage_bytes(int num_units, int n_rep, int head_dim) {
    if (num_units <= 0 || n_rep <= 0 || head_dim <= 0) return 0;
    // q and out at 4 bytes per element whatever the dtypes, new K and V likewise
    return (size_t)num_units * head_dim * (2 * (size_t)n_rep + 2) * 4;
}

extern "C" int kivi_decode_step_host(const kivi_layer* L, int64_t* quant_len, int* res_start, int* res_len,
                                     const void* h_q, const void* h_new_k, const void* h_new_v, void* h_out,
                                     int dtype, int out_dtype, int n_rep, float sm_scale,
                                     void* d_stage, size_t d_stage_bytes, void* workspace, size_t workspace_bytes,
                                     int num_splits, int path, int rounding, int chunks, int direct,
                                     const kivi_peer_gather* gather, int64_t gather_units, void* stream) {
    KIVI_REQUIRE(L && quant_len && res_start && res_len, "layer and counters must be given");
    KIVI_REQUIRE(h_q && h_new_k && h_new_v && h_out && workspace, "host and workspace buffers must be given");
    KIVI_REQUIRE(direct || d_stage, "a staging buffer is needed unless direct access is asked for");
    KIVI_REQUIRE(gather == nullptr || gather->epoch_dev == nullptr,
                 "the gathered rows are copied back from the buffer the host names: use a host-kept epoch here");
    KIVI_REQUIRE(dtype == KIVI_F32 || dtype == KIVI_BF16, "dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(out_dtype == KIVI_F32 || out_dtype == KIVI_BF16, "out dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(n_rep >= 1 && n_rep <= 8, "n_rep (%d) outside 1..8", n_rep);
    const int U = L->num_units, D = L->head_dim;
    KIVI_REQUIRE(U > 0 && D > 0, "empty layer");
    KIVI_REQUIRE(direct || d_stage_bytes >= kivi_decode_step_stage_bytes(U, n_rep, D), "staging buffer too small: %zu bytes given, %zu needed",
                 d_stage_bytes, kivi_decode_step_stage_bytes(U, n_rep, D));
    if (direct) {
        // device-side addresses of the pinned host buffers
        void *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
        KIVI_CUDA_OK(cudaHostGetDevicePointer(&dq, const_cast<void*>(h_q), 0));
        KIVI_CUDA_OK(cudaHostGetDevicePointer(&dk, const_cast<void*>(h_new_k), 0));
        KIVI_CUDA_OK(cudaHostGetDevicePointer(&dv, const_cast<void*>(h_new_v), 0));
        KIVI_CUDA_OK(cudaHostGetDevicePointer(&dout, h_out, 0));
        int64_t ql_d = 0; int rs_d = 0, rl_d = 0;
        if (int rc = kivi_cache_update(L, *quant_len, *res_start, *res_len, dk, dv, dtype, D, D, D, D, 1, rounding,
                                       &ql_d, &rs_d, &rl_d, stream)) return rc;
        int n_launch = kivi_last_launch_count();
        if (gather) {
            if (int rc = kivi_decode_attention_gather(L, ql_d, rs_d, rl_d, dq, dtype, gather, out_dtype, n_rep, sm_scale,
                                                      workspace, workspace_bytes, num_splits, path, stream)) return rc;
            KIVI_CUDA_OK(cudaMemcpyAsync(h_out, gather->out_ptrs[gather->rank], (size_t)gather_units * n_rep * D * elem_size(out_dtype),
                                         cudaMemcpyDeviceToHost, (cudaStream_t)stream));
        } else {
            if (int rc = kivi_decode_attention(L, ql_d, rs_d, rl_d, dq, dtype, dout, out_dtype, n_rep, sm_scale,
                                               workspace, workspace_bytes, num_splits, path, stream)) return rc;
        }
        n_launch += kivi_last_launch_count();
        *quant_len = ql_d; *res_start = rs_d; *res_len = rl_d;
        note_launches(n_launch);
        return KIVI_OK;
    }
    if (chunks < 1) chunks = 1;
    if (chunks > kMaxChunks) chunks = kMaxChunks;
    if (chunks > U) chunks = U;
    if (gather) chunks = 1;                        // the fused exchange counts one grid per call
    const size_t esz = elem_size(dtype), osz = elem_size(out_dtype);
    uint8_t* d_q = reinterpret_cast<uint8_t*>(d_stage);
    uint8_t* d_k = d_q + (size_t)U * n_rep * D * 4;
    uint8_t* d_v = d_k + (size_t)U * D * 4;
    uint8_t* d_o = d_v + (size_t)U * D * 4;
    cudaStream_t st = (cudaStream_t)stream;
    SideStreams* ss = nullptr;
    if (chunks > 1) {
        if (int rc = side_streams(&ss)) return rc;
        KIVI_CUDA_OK(cudaEventRecord(ss->fork, st));
    }
    int64_t ql = *quant_len; int rs = *res_start, rl = *res_len;
    int launches = 0;
    const size_t ws_per_unit = workspace_bytes / (size_t)U / 16 * 16;
    for (int c = 0; c < chunks; ++c) {
        const int u0 = (int)((int64_t)U * c / chunks), u1 = (int)((int64_t)U * (c + 1) / chunks), n = u1 - u0;
        cudaStream_t s = c == 0 ? st : ss->side[c - 1];
        if (c > 0) KIVI_CUDA_OK(cudaStreamWaitEvent(s, ss->fork, 0));
        const size_t qo = (size_t)u0 * n_rep * D, ko = (size_t)u0 * D;
        KIVI_CUDA_OK(cudaMemcpyAsync(d_q + qo * esz, reinterpret_cast<const uint8_t*>(h_q) + qo * esz, (size_t)n * n_rep * D * esz, cudaMemcpyHostToDevice, s));
        KIVI_CUDA_OK(cudaMemcpyAsync(d_k + ko * esz, reinterpret_cast<const uint8_t*>(h_new_k) + ko * esz, (size_t)n * D * esz, cudaMemcpyHostToDevice, s));
        KIVI_CUDA_OK(cudaMemcpyAsync(d_v + ko * esz, reinterpret_cast<const uint8_t*>(h_new_v) + ko * esz, (size_t)n * D * esz, cudaMemcpyHostToDevice, s));
        kivi_layer Lc = slice_units(L, u0, u1);
        int64_t ql_c = 0; int rs_c = 0, rl_c = 0;
        if (int rc = kivi_cache_update(&Lc, *quant_len, *res_start, *res_len, d_k + ko * esz, d_v + ko * esz, dtype,
                                       D, D, D, D, 1, rounding, &ql_c, &rs_c, &rl_c, s)) return rc;
        launches += kivi_last_launch_count();
        ql = ql_c; rs = rs_c; rl = rl_c;
        void* ws_c = reinterpret_cast<uint8_t*>(workspace) + ws_per_unit * u0;
        if (gather) {
            if (int rc = kivi_decode_attention_gather(&Lc, ql_c, rs_c, rl_c, d_q + qo * esz, dtype, gather, out_dtype, n_rep, sm_scale,
                                                      ws_c, ws_per_unit * n, num_splits, path, s)) return rc;
            launches += kivi_last_launch_count();
            KIVI_CUDA_OK(cudaMemcpyAsync(h_out, gather->out_ptrs[gather->rank], (size_t)gather_units * n_rep * D * osz, cudaMemcpyDeviceToHost, s));
        } else {
            if (int rc = kivi_decode_attention(&Lc, ql_c, rs_c, rl_c, d_q + qo * esz, dtype, d_o + qo * osz, out_dtype, n_rep, sm_scale,
                                               ws_c, ws_per_unit * n, num_splits, path, s)) return rc;
            launches += kivi_last_launch_count();
            KIVI_CUDA_OK(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(h_out) + qo * osz, d_o + qo * osz, (size_t)n * n_rep * D * osz, cudaMemcpyDeviceToHost, s));
        }
        if (c > 0) {
            KIVI_CUDA_OK(cudaEventRecord(ss->join[c - 1], s));
            KIVI_CUDA_OK(cudaStreamWaitEvent(st, ss->join[c - 1], 0));
        }
    }
    *quant_len = ql; *res_start = rs; *res_len = rl;
    note_launches(launches);
    return KIVI_OK;
}
