// extern "C" surface of libkivi_cuda: error state, operator wrappers, and the
// decode-attention dispatcher (split planning, workspace carve-up, merge).
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include "kivi_common.cuh"

namespace kivi {

static thread_local char g_err[512] = "";
static thread_local int g_launches = 0;

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

void note_launches(int n) { g_launches = n; }

int num_sms() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

constexpr int kMaxSplitsC = 128;

int run_group_quant(const void* in, int in_dtype, uint8_t* packed, float* scales, float* zeros,
                    float* rt, int64_t num_groups, int G, int rounding, int mode, cudaStream_t st);
int run_group_dequant(const uint8_t* packed, const float* scales, const float* zeros, float* out,
                      int64_t num_groups, int G, cudaStream_t st);
int validate_layer(const kivi_layer* L);
int validate_state(const kivi_layer* L, int64_t quant_len, int res_start, int res_len);
int run_attn_fp32(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                  const void* q, int q_dtype, int n_rep, float scale_log2, int nq_splits, int gps,
                  int n_splits, float* part_o, float* part_ml, cudaStream_t st);
bool attn_mma_supported(const kivi_layer* L, int n_rep, const void* q);
void attn_mma_residual_plan(int res_len, int* n_res_splits, int* res_chunk);
int attn_mma_ctas_per_sm();
int run_attn_mma(const kivi_layer* L, int64_t quant_len, int res_start, int res_len,
                 const void* q, int q_dtype, int n_rep, float scale_log2, int nq_splits, int gps,
                 int n_res_splits, int res_chunk, float* part_o, float* part_ml, cudaStream_t st);
int run_sample(const void* logits, int dtype, int batch, int vocab, int64_t row_stride, float temperature, int top_k,
               int do_sample, uint64_t seed, uint64_t step, int64_t* ids, cudaStream_t st);
int run_merge_token_shards(const float* parts, int n_shards, int64_t rows, int D, void* out, int out_dtype,
                           float* lse_out, cudaStream_t st);
int run_mma_alignment_probe(int* bits_out);
int attn_mma_fault_word(int* out);
int gather_fault_word(int* out);
int attn_mma_fault_clear();
int gather_fault_clear();
int run_merge(const float* part_o, const float* part_ml, void* out, const kivi_peer_gather* gather, float* lse,
              int out_dtype, int num_units, int n_rep, int n_splits, int D, cudaStream_t st);

}  // namespace kivi

using namespace kivi;

extern "C" const char* kivi_last_error(void) { return g_err; }
extern "C" int kivi_version(void) { return 100; }
extern "C" int kivi_last_launch_count(void) { return g_launches; }
extern "C" int kivi_device_fault(int* word_out) {
    KIVI_REQUIRE(word_out != nullptr, "word_out is null");
    int copy_wait = 0, peer_wait = 0;
    if (int rc = attn_mma_fault_word(&copy_wait)) return rc;
    if (int rc = gather_fault_word(&peer_wait)) return rc;
    *word_out = (copy_wait ? 1 : 0) | (peer_wait ? 2 : 0);
    return KIVI_OK;
}

extern "C" int kivi_device_fault_clear(void) {
    if (int rc = attn_mma_fault_clear()) return rc;
    return gather_fault_clear();
}

static int check_values_args(int64_t num_tokens, int head_dim, int group_size) {
    KIVI_REQUIRE(group_size > 0 && group_size % 4 == 0, "group_size must be positive and divisible by 4");
    KIVI_REQUIRE(head_dim > 0 && head_dim % group_size == 0, "head_dim must be positive and divisible by group_size");
    KIVI_REQUIRE(num_tokens > 0, "input must be non-empty");
    return KIVI_OK;
}

extern "C" int kivi_quantize_keys_per_channel(const void* input, int in_dtype, uint8_t* output,
                                              float* scales, float* zeros, int64_t num_channels,
                                              int group_size, int rounding, void* stream) {
    return run_group_quant(input, in_dtype, output, scales, zeros, nullptr, num_channels, group_size,
                           rounding, 0, (cudaStream_t)stream);
}

extern "C" int kivi_quantize_values_per_token(const void* input, int in_dtype, uint8_t* output,
                                              float* scales, float* zeros, int64_t num_tokens,
                                              int head_dim, int group_size, int rounding, void* stream) {
    if (int rc = check_values_args(num_tokens, head_dim, group_size)) return rc;
    return run_group_quant(input, in_dtype, output, scales, zeros, nullptr,
                           num_tokens * (head_dim / group_size), group_size, rounding, 0, (cudaStream_t)stream);
}

extern "C" int kivi_dequantize_keys_per_channel(const uint8_t* input, const float* scales,
                                                const float* zeros, float* output,
                                                int64_t num_channels, int group_size, void* stream) {
    return run_group_dequant(input, scales, zeros, output, num_channels, group_size, (cudaStream_t)stream);
}

extern "C" int kivi_dequantize_values_per_token(const uint8_t* input, const float* scales,
                                                const float* zeros, float* output,
                                                int64_t num_groups, int group_size, void* stream) {
    return run_group_dequant(input, scales, zeros, output, num_groups, group_size, (cudaStream_t)stream);
}

extern "C" int kivi_quant_dequant_roundtrip_keys(const void* input, int in_dtype, float* output,
                                                 int64_t num_channels, int group_size, int rounding,
                                                 void* stream) {
    return run_group_quant(input, in_dtype, nullptr, nullptr, nullptr, output, num_channels, group_size,
                           rounding, 1, (cudaStream_t)stream);
}

extern "C" int kivi_quant_dequant_roundtrip_values(const void* input, int in_dtype, float* output,
                                                   int64_t num_tokens, int head_dim, int group_size,
                                                   int rounding, void* stream) {
    if (int rc = check_values_args(num_tokens, head_dim, group_size)) return rc;
    return run_group_quant(input, in_dtype, nullptr, nullptr, nullptr, output,
                           num_tokens * (head_dim / group_size), group_size, rounding, 1, (cudaStream_t)stream);
}

// ---- decode attention ------------------------------------------------------

extern "C" int kivi_decode_attention_max_splits(void) { return kMaxSplitsC; }

// partial outputs [units][splits+8][n_rep][D] + (max, sum) [units][splits+8][n_rep][2];
// the +8 covers the residual-ring parts (1 for the fp32 kernel, up to 8 for the
// tensor-core kernel).
extern "C" size_t kivi_decode_attention_workspace(int num_units, int n_rep, int head_dim, int num_splits) {
    if (num_units <= 0 || n_rep <= 0 || head_dim <= 0) return 0;
    if (num_splits <= 0 || num_splits > kMaxSplitsC) num_splits = kMaxSplitsC;
    return (size_t)num_units * (num_splits + 8) * n_rep * (head_dim + 2) * sizeof(float);
}

static int clamp_splits(int64_t s, int64_t n_groups) {
    if (s > kMaxSplitsC) s = kMaxSplitsC;
    if (s > n_groups) s = n_groups;
    if (s < 1) s = 1;
    return (int)s;
}

// CUDA-core kernel: aim at ~8 CTAs of 128 threads per SM, never below 4 token
// groups per CTA.
static int plan_splits_fp32(int num_units, int64_t n_groups, int requested) {
    if (n_groups <= 0) return 0;
    if (requested > 0) return clamp_splits(requested, n_groups);
    const int64_t target = (int64_t)num_sms() * 8;
    int64_t s = (target + num_units - 1) / num_units;
    const int64_t cap = (n_groups + 3) / 4;
    if (s > cap) s = cap;
    return clamp_splits(s, n_groups);
}

// Tensor-core kernel: how many pieces to cut every unit's quantized history into.
// Evaluates a small cost model for every candidate count and keeps the cheapest
// (ties: fewer pieces).  `slots` CTAs are resident at a time (SMs x CTAs per SM).
// Constants in microseconds, fitted to CUDA-event times on B200 at about 1.9 GHz
// (units x tokens from 1 x 128k and 16 x 1k to 512 x 32k): a CTA costs c0 of
// fixed time (first copy, query staging, the fold of its warps) plus c1 per token
// group, a residual-ring CTA t_ring, starting a CTA c_start, folding the pieces
// of a unit c_fold.  c1 depends on how many CTAs share an SM (an SM with three
// CTAs delivers 8.3-9 groups per us, with two 7.4-8, with one 5.7-6): 0.16 /
// 0.24 / 0.33 us per group for a single wave with at most 1 / 2 / 3 quantized
// CTAs per SM, 0.36 in the steady state of several waves.  The fold of more
// than 16 pieces is done by a whole CTA per output row and costs less per
// piece.  The grid lists the
// quantized pieces first and the short ring CTAs last, so:
//   * the quantized CTAs all resident at once: the time of one of them (the ring
//     CTAs fill the free slots, or follow the first ring CTAs that finish);
//   * several waves: total CTA time over the slots, plus a ragged end of about
//     a third of a CTA.
static int plan_splits_mma(int num_units, int64_t n_groups, int requested, int n_res_splits, int sms, int ctas_per_sm) {
    if (n_groups <= 0) return 0;
    if (requested > 0) return clamp_splits(requested, n_groups);
    const int n_sms = sms > 0 ? sms : 148, per_sm = ctas_per_sm > 0 ? ctas_per_sm : 3;
    const double slots = (double)per_sm * n_sms;
    const double c0 = 6.0, c1_one = 0.16, c1_two = 0.24, c1_three = 0.33, c1_full = 0.36;
    const double t_ring = 7.0, c_start = 0.015, ragged = 0.3;
    const int64_t s_max = n_groups < kMaxSplitsC ? n_groups : kMaxSplitsC;
    int best = 1;
    double best_t = 0.0;
    for (int64_t s = 1; s <= s_max; ++s) {
        const double quant = (double)num_units * (double)s, ring = (double)num_units * n_res_splits;
        const double per_cta = (double)((n_groups + s - 1) / s);
        double t;
        if (quant <= slots) {
            // the fullest SM sets the pace.  The two-CTA rate only holds up to about
            // 1.75 CTAs per SM on average: with 288 or 296 CTAs on 148 SMs a CTA was
            // measured at 0.27-0.32 us per group, as if some SMs already held three.
            const double c1 = quant <= n_sms ? c1_one : quant <= 1.75 * n_sms ? c1_two : quant <= 3.0 * n_sms ? c1_three : c1_full;
            t = c0 + c1 * per_cta + c_start * (quant + ring);
        } else {
            t = (quant * (c0 + c1_full * per_cta) + ring * t_ring) / slots + ragged * (c0 + c1_full * per_cta);
            // just over one wave: never cheaper than a full single wave of such CTAs
            const double one_wave = c0 + c1_three * per_cta + c_start * slots;
            if (t < one_wave) t = one_wave;
        }
        t += s <= 16 ? 0.1 * (double)s : 1.0 + 0.02 * (double)s;
        if (s == 1 || t < best_t - 1e-9) { best = (int)s; best_t = t; }
    }
    return best;
}

extern "C" int kivi_decode_attention_plan(int num_units, int64_t quant_len, int res_len, int head_dim, int group_size,
                                          int n_rep, int q_dtype, int num_splits, int path, int sms, int ctas_per_sm,
                                          int* tensor_cores_out, int* quant_splits_out, int* residual_parts_out) {
    KIVI_REQUIRE(num_units > 0 && head_dim > 0 && group_size > 0 && quant_len >= 0 && quant_len % group_size == 0 && res_len >= 0,
                 "invalid shape");
    KIVI_REQUIRE(num_splits >= 0 && num_splits <= kMaxSplitsC, "num_splits (%d) outside 0..%d", num_splits, kMaxSplitsC);
    KIVI_REQUIRE(tensor_cores_out && quant_splits_out && residual_parts_out, "output pointers must be given");
    const bool shape_ok = head_dim == 128 && group_size == 32 && n_rep >= 1 && n_rep <= 8;
    const bool use_mma = path == KIVI_ATTN_MMA ? shape_ok : path == KIVI_ATTN_AUTO ? (shape_ok && q_dtype == KIVI_BF16) : false;
    if (path == KIVI_ATTN_MMA && !shape_ok) {
        set_error("tensor-core path needs head_dim 128, group_size 32, n_rep <= 8 (got %d, %d, %d)", head_dim, group_size, n_rep);
        return KIVI_ERR_UNSUPPORTED;
    }
    int n_res = res_len > 0 ? 1 : 0, chunk = res_len;
    if (use_mma) attn_mma_residual_plan(res_len, &n_res, &chunk);
    const int64_t n_groups = quant_len / group_size;
    if (sms <= 0) sms = num_sms();
    if (ctas_per_sm <= 0) ctas_per_sm = attn_mma_ctas_per_sm();
    *tensor_cores_out = use_mma ? 1 : 0;
    *quant_splits_out = use_mma ? plan_splits_mma(num_units * ((n_rep + 3) / 4), n_groups, num_splits, n_res, sms, ctas_per_sm)
                                : plan_splits_fp32(num_units, n_groups, num_splits);
    *residual_parts_out = n_res;
    return KIVI_OK;
}

static int decode_attention_impl(const kivi_layer* L, int64_t quant_len, int res_start,
                                 int res_len, const void* q, int q_dtype, void* out,
                                 const kivi_peer_gather* gather, float* lse, int out_dtype,
                                 int n_rep, float sm_scale, void* workspace, size_t workspace_bytes,
                                 int num_splits, int path, void* stream) {
    if (int rc = validate_layer(L)) return rc;
    if (int rc = validate_state(L, quant_len, res_start, res_len)) return rc;
    KIVI_REQUIRE(q && (out || gather), "q / out are null");
    KIVI_REQUIRE(q_dtype == KIVI_F32 || q_dtype == KIVI_BF16, "q dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(out_dtype == KIVI_F32 || out_dtype == KIVI_BF16, "out dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(n_rep >= 1 && n_rep <= 8, "n_rep (%d) outside 1..8", n_rep);
    KIVI_REQUIRE(quant_len + res_len > 0, "the cache is empty: nothing to attend to");
    KIVI_REQUIRE(num_splits >= 0 && num_splits <= kMaxSplitsC, "num_splits (%d) outside 0..%d", num_splits, kMaxSplitsC);
    KIVI_REQUIRE(path == KIVI_ATTN_AUTO || path == KIVI_ATTN_FP32 || path == KIVI_ATTN_MMA, "unknown path %d", path);
    KIVI_REQUIRE(L->num_units <= 65535, "num_units (%d) above 65535", L->num_units);
    const int D = L->head_dim, G = L->group_size;
    const int64_t n_groups = quant_len / G;
    bool use_mma = false;
    if (path == KIVI_ATTN_MMA) {
        if (!attn_mma_supported(L, n_rep, q)) {
            set_error("tensor-core path needs head_dim 128, group_size 32, n_rep <= 8 (got %d, %d, %d) and 16-byte aligned arrays", D, G, n_rep);
            return KIVI_ERR_UNSUPPORTED;
        }
        use_mma = true;
    } else if (path == KIVI_ATTN_AUTO) {
        // fp32 queries keep the all-fp32 kernel (1e-5 tolerance); bf16 queries take
        // the tensor-core kernel when the shape allows it
        use_mma = q_dtype == KIVI_BF16 && attn_mma_supported(L, n_rep, q);
    }
    int n_res_splits = res_len > 0 ? 1 : 0, res_chunk = res_len;
    if (use_mma) attn_mma_residual_plan(res_len, &n_res_splits, &res_chunk);
    const int nq_splits = use_mma ? plan_splits_mma(L->num_units * ((n_rep + 3) / 4), n_groups, num_splits, n_res_splits, num_sms(), attn_mma_ctas_per_sm())
                                  : plan_splits_fp32(L->num_units, n_groups, num_splits);
    const int gps = nq_splits > 0 ? (int)((n_groups + nq_splits - 1) / nq_splits) : 0;
    const int n_splits = nq_splits + n_res_splits;
    const size_t need = (size_t)L->num_units * n_splits * n_rep * (D + 2) * sizeof(float);
    KIVI_REQUIRE(workspace != nullptr && workspace_bytes >= need,
                 "workspace too small: %zu bytes given, %zu needed", workspace_bytes, need);
    KIVI_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15u) == 0, "workspace must be 16-byte aligned");
    float* part_o = reinterpret_cast<float*>(workspace);
    float* part_ml = part_o + (size_t)L->num_units * n_splits * n_rep * D;
    if (sm_scale <= 0.0f) sm_scale = 1.0f / sqrtf((float)D);
    const float scale_log2 = sm_scale * 1.4426950408889634f;
    cudaStream_t st = (cudaStream_t)stream;

    int rc = use_mma
        ? run_attn_mma(L, quant_len, res_start, res_len, q, q_dtype, n_rep, scale_log2, nq_splits, gps, n_res_splits, res_chunk, part_o, part_ml, st)
        : run_attn_fp32(L, quant_len, res_start, res_len, q, q_dtype, n_rep, scale_log2, nq_splits, gps, n_splits, part_o, part_ml, st);
    if (rc) return rc;
    if (int rc2 = run_merge(part_o, part_ml, out, gather, lse, out_dtype, L->num_units, n_rep, n_splits, D, st)) return rc2;
    note_launches(2);
    return KIVI_OK;
}

extern "C" int kivi_decode_attention(const kivi_layer* L, int64_t quant_len, int res_start,
                                     int res_len, const void* q, int q_dtype, void* out, int out_dtype,
                                     int n_rep, float sm_scale, void* workspace, size_t workspace_bytes,
                                     int num_splits, int path, void* stream) {
    return decode_attention_impl(L, quant_len, res_start, res_len, q, q_dtype, out, nullptr, nullptr, out_dtype, n_rep,
                                 sm_scale, workspace, workspace_bytes, num_splits, path, stream);
}

extern "C" int kivi_decode_attention_lse(const kivi_layer* L, int64_t quant_len, int res_start,
                                         int res_len, const void* q, int q_dtype, void* out, int out_dtype,
                                         float* lse_out, int n_rep, float sm_scale, void* workspace,
                                         size_t workspace_bytes, int num_splits, int path, void* stream) {
    KIVI_REQUIRE(lse_out != nullptr, "lse_out is null");
    KIVI_REQUIRE(quant_len + res_len > 0, "the log-sum-exp of an empty cache is undefined");
    return decode_attention_impl(L, quant_len, res_start, res_len, q, q_dtype, out, nullptr, lse_out, out_dtype, n_rep,
                                 sm_scale, workspace, workspace_bytes, num_splits, path, stream);
}

// ---- decode attention + all-gather over peer memory -------------------------------
extern "C" int kivi_decode_attention_gather(const kivi_layer* L, int64_t quant_len, int res_start,
                                            int res_len, const void* q, int q_dtype,
                                            const kivi_peer_gather* gather, int out_dtype,
                                            int n_rep, float sm_scale, void* workspace, size_t workspace_bytes,
                                            int num_splits, int path, void* stream) {
    KIVI_REQUIRE(gather != nullptr, "gather is null");
    KIVI_REQUIRE(gather->world >= 1 && gather->world <= KIVI_PEER_MAX_WORLD, "world (%d) outside 1..%d", gather->world, KIVI_PEER_MAX_WORLD);
    KIVI_REQUIRE(gather->rank >= 0 && gather->rank < gather->world, "rank (%d) outside 0..%d", gather->rank, gather->world - 1);
    KIVI_REQUIRE(gather->unit_offset >= 0, "unit_offset is negative");
    KIVI_REQUIRE(gather->epoch_dev != nullptr || gather->epoch != 0, "epoch starts at 1");
    KIVI_REQUIRE(gather->epoch_dev == nullptr || gather->alt_bytes > 0, "a device-kept epoch needs the distance between the two buffers (alt_bytes)");
    for (int r = 0; r < gather->world; ++r)
        KIVI_REQUIRE(gather->out_ptrs[r] != nullptr && gather->flag_ptrs[r] != nullptr, "buffer or flag pointer of rank %d is null", r);
    return decode_attention_impl(L, quant_len, res_start, res_len, q, q_dtype, nullptr, gather, nullptr, out_dtype, n_rep,
                                 sm_scale, workspace, workspace_bytes, num_splits, path, stream);
}

// Inter-process buffers for the gather: plain cudaMalloc memory shared through
// CUDA IPC handles (same node; the driver maps the peer's memory over NVLink).
extern "C" int kivi_peer_alloc(size_t bytes, void** ptr_out, unsigned char handle_out[64]) {
    KIVI_REQUIRE(bytes > 0 && ptr_out != nullptr && handle_out != nullptr, "bytes, ptr_out and handle_out must be given");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    void* p = nullptr;
    KIVI_CUDA_OK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        set_error("kivi_peer_alloc failed: %s", cudaGetErrorString(e));
        return KIVI_ERR_CUDA;
    }
    memcpy(handle_out, &h, 64);
    *ptr_out = p;
    return KIVI_OK;
}

extern "C" int kivi_peer_open(const unsigned char handle[64], void** ptr_out) {
    KIVI_REQUIRE(handle != nullptr && ptr_out != nullptr, "handle and ptr_out must be given");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    KIVI_CUDA_OK(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return KIVI_OK;
}

extern "C" int kivi_peer_close(void* ptr) {
    KIVI_REQUIRE(ptr != nullptr, "ptr is null");
    KIVI_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return KIVI_OK;
}

extern "C" int kivi_peer_free(void* ptr) {
    KIVI_REQUIRE(ptr != nullptr, "ptr is null");
    KIVI_CUDA_OK(cudaFree(ptr));
    return KIVI_OK;
}

// ---- decode attention without a caller workspace --------------------------------
// The split partials of this entry point live in a fixed array in the library
// image instead of caller memory, for hosts that may not allocate (see the
// header).  `g_noalloc_scratch` is a device symbol: in host code the name is not
// a device address, so the address is looked up once per device with
// cudaGetSymbolAddress and cached.
static __device__ __align__(256) unsigned char g_noalloc_scratch[KIVI_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" int kivi_decode_attention_noalloc(const kivi_layer* L, int64_t quant_len, int res_start,
                                             int res_len, const void* q, int q_dtype, void* out,
                                             int out_dtype, int n_rep, float sm_scale, int num_splits,
                                             int path, void* stream) {
    int dev = 0;
    KIVI_CUDA_OK(cudaGetDevice(&dev));
    KIVI_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d outside 0..%d", dev, kMaxDevices - 1);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_ptr[dev] == nullptr) {
            void* p = nullptr;
            KIVI_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch));   // this device's copy of the array
            g_noalloc_ptr[dev] = p;
        }
        scratch = g_noalloc_ptr[dev];
    }
    const int rc = kivi_decode_attention(L, quant_len, res_start, res_len, q, q_dtype, out, out_dtype, n_rep,
                                         sm_scale, scratch, (size_t)KIVI_NOALLOC_SCRATCH_BYTES, num_splits, path, stream);
    if (rc == KIVI_ERR_INVALID_ARGUMENT && strstr(g_err, "workspace too small") != nullptr) {
        char detail[256];
        strncpy(detail, g_err, sizeof(detail) - 1);          // the message above is far shorter than this
        detail[sizeof(detail) - 1] = 0;
        set_error("problem too large for the built-in scratch of kivi_decode_attention_noalloc (%u bytes): %s; "
                  "pass a smaller num_splits or call kivi_decode_attention with your own workspace",
                  (unsigned)KIVI_NOALLOC_SCRATCH_BYTES, detail);
    }
    return rc;
}

// ---- next-token choice -----------------------------------------------------------
extern "C" int kivi_sample_tokens(const void* logits, int dtype, int batch, int vocab, int64_t row_stride,
                                  float temperature, int top_k, int do_sample, uint64_t seed, uint64_t step,
                                  int64_t* ids_out, void* stream) {
    KIVI_REQUIRE(logits != nullptr && ids_out != nullptr, "logits / ids_out are null");
    KIVI_REQUIRE(dtype == KIVI_F32 || dtype == KIVI_BF16, "logits dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(batch > 0 && vocab > 0 && row_stride >= vocab, "batch (%d), vocab (%d) and row_stride must be positive, row_stride >= vocab", batch, vocab);
    KIVI_REQUIRE(top_k >= 0, "top_k (%d) is negative; 0 means no cut", top_k);
    return run_sample(logits, dtype, batch, vocab, row_stride, temperature, top_k, do_sample, seed, step, ids_out,
                      (cudaStream_t)stream);
}

// ---- sequence sharding: fold per-shard (output, log-sum-exp) rows ----------------------
extern "C" int kivi_merge_token_shards(const float* parts, int n_shards, int64_t rows, int head_dim, void* out,
                                       int out_dtype, float* lse_out, void* stream) {
    KIVI_REQUIRE(parts != nullptr && out != nullptr, "parts / out are null");
    KIVI_REQUIRE(n_shards >= 1 && rows >= 1 && head_dim >= 1, "n_shards, rows and head_dim must be positive");
    KIVI_REQUIRE(out_dtype == KIVI_F32 || out_dtype == KIVI_BF16, "out dtype must be KIVI_F32 or KIVI_BF16");
    KIVI_REQUIRE(rows < ((int64_t)1 << 33), "too many rows");
    if (int rc = run_merge_token_shards(parts, n_shards, rows, head_dim, out, out_dtype, lse_out, (cudaStream_t)stream)) return rc;
    note_launches(1);
    return KIVI_OK;
}

// ---- self-test of a hardware property the tensor-core kernel's error budget rests on ----
extern "C" int kivi_selftest_mma_alignment_bits(int* bits_out) {
    KIVI_REQUIRE(bits_out != nullptr, "bits_out is null");
    return run_mma_alignment_probe(bits_out);
}
