/*
 * kivi_cuda.h — C ABI of libkivi_cuda.so, the B200 (sm_100a) implementation of
 * the KIVI 2-bit KV-cache hot path.
 *
 * Plain pointers and sizes only; every pointer marked "device" must be CUDA
 * device memory on the current device; `stream` is a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  Every entry point validates its
 * arguments on the host, enqueues its kernels on `stream` and returns without
 * synchronising.  Return value: KIVI_OK or a KIVI_ERR_* code;
 * kivi_last_error() gives the message of the calling thread's last failure.
 * There is no CPU fallback anywhere in this library.
 *
 * "reference" below = the kivi_sycl project this library is a drop-in for;
 * citations are path:line inside that project.
 */
#ifndef KIVI_CUDA_H_
#define KIVI_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KIVI_OK 0
#define KIVI_ERR_INVALID_ARGUMENT 1 /* host-side validation failed, nothing launched */
#define KIVI_ERR_CUDA 2             /* a CUDA runtime call failed */
#define KIVI_ERR_UNSUPPORTED 3      /* valid arguments this build has no kernel for */

/* element types of activations (inputs, queries, residual window, outputs) */
#define KIVI_F32 0
#define KIVI_BF16 1

/* how (x-min)/scale exactly halfway between two codes is rounded.
 * HALF_AWAY is what the reference's device kernel does (sycl::round,
 * src/csrc/kernels/internal/quant_tile.hpp:64,85); HALF_EVEN is what the
 * reference's torch mirror does (torch.round, examples/cpu_sim.py:42). */
#define KIVI_ROUND_HALF_AWAY 0
#define KIVI_ROUND_HALF_EVEN 1

const char* kivi_last_error(void);
int kivi_version(void); /* major*10000 + minor*100 + patch */

/* ------------------------------------------------------------------------
 * Operators on the flat packed layout of the reference.
 *
 * Every operator works on consecutive runs of `group_size` elements of the
 * flat input: run g gives scales[g] = (max-min)/3.0f + 1e-10f, zeros[g] = min,
 * and group_size/4 bytes q0|q1<<2|q2<<4|q3<<6 with
 * q = clamp(round((x-min)/scale), 0, 3).  Dequantize is float(q)*scale+zero
 * with a separate multiply and add.  in_dtype KIVI_BF16 upcasts each element
 * to fp32 first (the reference upcasts with .float(), cache/manager.py:210-214).
 * group_size must be a positive multiple of 4.
 * ---------------------------------------------------------------------- */

/* replaces quantize_keys_per_channel_submit, src/csrc/kernels/quantize_kernels.cpp:24-54
 * input  device [num_channels*group_size] (keys transposed to [B,H,D,S], groups along S)
 * output device [num_channels*group_size/4] u8; scales, zeros device [num_channels] f32 */
int kivi_quantize_keys_per_channel(const void* input, int in_dtype, uint8_t* output,
                                   float* scales, float* zeros, int64_t num_channels,
                                   int group_size, int rounding, void* stream);

/* replaces quantize_values_per_token_submit, src/csrc/kernels/quantize_kernels.cpp:69-106
 * input device [num_tokens*head_dim]; output [num_tokens*head_dim/4];
 * scales, zeros [num_tokens*head_dim/group_size]; head_dim % group_size == 0 */
int kivi_quantize_values_per_token(const void* input, int in_dtype, uint8_t* output,
                                   float* scales, float* zeros, int64_t num_tokens,
                                   int head_dim, int group_size, int rounding, void* stream);

/* replaces dequantize_keys_per_channel_submit, src/csrc/kernels/dequantize_kernels.cpp:32-64 */
int kivi_dequantize_keys_per_channel(const uint8_t* input, const float* scales,
                                     const float* zeros, float* output,
                                     int64_t num_channels, int group_size, void* stream);

/* replaces dequantize_values_per_token_submit, src/csrc/kernels/dequantize_kernels.cpp:79-111 */
int kivi_dequantize_values_per_token(const uint8_t* input, const float* scales,
                                     const float* zeros, float* output,
                                     int64_t num_groups, int group_size, void* stream);

/* replaces quant_dequant_roundtrip_keys_submit, src/csrc/kernels/roundtrip_kernels.cpp:14-38 */
int kivi_quant_dequant_roundtrip_keys(const void* input, int in_dtype, float* output,
                                      int64_t num_channels, int group_size, int rounding,
                                      void* stream);

/* replaces quant_dequant_roundtrip_values_submit, src/csrc/kernels/roundtrip_kernels.cpp:50-80 */
int kivi_quant_dequant_roundtrip_values(const void* input, int in_dtype, float* output,
                                        int64_t num_tokens, int head_dim, int group_size,
                                        int rounding, void* stream);

/* ------------------------------------------------------------------------
 * Device-resident cache of one layer on one GPU.
 *
 * Replaces the storage side of KiviCache (src/kivi_sycl/cache/manager.py:100-117):
 * the reference keeps an fp32 residual on the CPU and a dequantized fp32
 * history; here the residual is a ring in device memory and the history is
 * kept packed.  A "unit" is one (batch, kv_head) pair; units are independent.
 *
 * Quantized store of one unit, token group g (tokens g*G .. g*G+G-1):
 *   k_codes  + (u*max_groups + g) * (D*G/4): one key block.  With Q = G/4 and
 *            W = min(D,64), the byte at  (d/W)*Q*W + j*W + p(d%W)  (0<=j<Q) holds
 *            the codes of channel d for tokens 4j .. 4j+3 of the group in bits
 *            0-1, 2-3, 4-5, 6-7 (the byte the reference's key operator writes);
 *            p is the identity for W < 64 and for W = 64 swaps bits 2-3 with
 *            bits 4-5 of its argument.
 *   k_scales, k_zeros + (u*max_groups + g) * D : fp32 per channel of the group
 *            (one per-channel group of the reference, quantize_kernels.hpp:36-42).
 *   v_codes  + (u*max_tokens + t) * (D/4): the reference's value layout, byte b
 *            = channels 4b..4b+3 of token t (quantize_kernels.hpp:55-60).
 *   v_scales, v_zeros + (u*max_tokens + t) * (D/G): fp32 per channel group.
 *            For D = 128, G = 32 the 32 token rows of a group are permuted
 *            inside the group's own 1 KB / 512 B: code byte b of token
 *            t = 16k + 4c + n is byte n of 32-bit word (b/8)*64 + k*32 + (b%8)*4 + c,
 *            and the token's scale/zero row is 16k + 4n + c.
 * Residual ring of one unit: k_res, v_res + u*R*D elements of res_dtype; the
 * live window is slots (res_start + i) % R for 0 <= i < res_len, oldest first.
 * The three counters (quant_len, res_start, res_len) are kept by the caller;
 * kivi_cache_update returns their new values and never reads device memory
 * back.
 * ---------------------------------------------------------------------- */
typedef struct kivi_layer {
    int32_t num_units;    /* B * Hkv held by this GPU */
    int32_t head_dim;     /* D; multiple of group_size; D <= 64 or D % 64 == 0 */
    int32_t group_size;   /* G; >= 4, multiple of 4 */
    int32_t residual_cap; /* R; >= G */
    int64_t max_tokens;   /* capacity of the quantized store, multiple of G */
    int32_t res_dtype;    /* KIVI_F32 or KIVI_BF16 */
    int32_t reserved;
    uint8_t* k_codes;
    float* k_scales;
    float* k_zeros;
    uint8_t* v_codes;
    float* v_scales;
    float* v_zeros;
    void* k_res;
    void* v_res;
} kivi_layer;

/* Flush policy of the reference (append everything, then move the oldest G
 * tokens to the quantized store while the window holds >= R tokens,
 * cache/manager.py:226-243).  Pure host arithmetic. */
int kivi_cache_plan(int64_t quant_len, int res_len, int n_new, int group_size,
                    int residual_cap, int* n_flush_groups, int64_t* quant_len_out,
                    int* res_len_out);

/* replaces KiviCache.add_tokens + _flush_group, cache/manager.py:162-249, 309-374.
 * new_k/new_v: device, n_new tokens per unit of new_dtype; token t of unit u at
 * element offset u*unit_stride + t*tok_stride, head_dim contiguous elements.
 * Groups are cut from the sequence [live ring tokens, then the new tokens],
 * keys quantized per channel over the G tokens of a group, values per token
 * over runs of G channels, written at group index quant_len/G onwards; what is
 * left goes to the ring.  Fails if the store would overflow. */
int kivi_cache_update(const kivi_layer* layer, int64_t quant_len, int res_start, int res_len,
                      const void* new_k, const void* new_v, int new_dtype,
                      int64_t unit_stride_k, int64_t tok_stride_k,
                      int64_t unit_stride_v, int64_t tok_stride_v, int n_new,
                      int rounding, int64_t* quant_len_out, int* res_start_out,
                      int* res_len_out, void* stream);

/* replaces the serving half of KiviCache.get_full_cache, cache/manager.py:251-290
 * (compatibility path; the attention below never needs it).  Writes fp32
 * [num_units][quant_len + res_len][D] keys and values: dequantized history
 * followed by the residual window in age order. */
int kivi_cache_materialize(const kivi_layer* layer, int64_t quant_len, int res_start,
                           int res_len, float* k_out, float* v_out, void* stream);

/* Re-lays keys quantized by kivi_quantize_keys_per_channel (channel-major
 * [num_units][D][S/4] codes, [num_units][D][S/G] scales and zeros, the layout of
 * README.md:122-128 with S/G groups per channel) into the key blocks of
 * `layer` at groups 0 .. S/G-1.  No reference counterpart: the reference never
 * keeps packed keys (cache/manager.py:100-109). */
int kivi_cache_import_keys(const kivi_layer* layer, const uint8_t* packed,
                           const float* scales, const float* zeros, int64_t seq_len,
                           void* stream);

/* ------------------------------------------------------------------------
 * Fused decode attention over the packed cache.
 *
 * No counterpart kernel in the reference: it serves a dequantized fp32 cache to
 * a third-party model (cache/manager.py:251-290, generation/generate.py:75-77)
 * and states the math once, tests/integration/test_attention_fix.py:40-43:
 *   out = softmax(q K^T * head_dim^-0.5) V  over  [history || residual].
 * q, out: device [num_units][n_rep][D] (n_rep = query heads per KV head; with
 * units ordered (b, kv_head) this is the contiguous [B, Hq, D] tensor).
 * sm_scale <= 0 means head_dim^-0.5.
 * workspace: device scratch of at least kivi_decode_attention_workspace()
 * bytes, holding split partials (running max, sum and unnormalised output per
 * split); contents need not be preserved between calls.
 * num_splits: how many pieces the quantized history of a unit is cut into;
 * 0 = choose from the SM count.  path: KIVI_ATTN_AUTO picks the tensor-core
 * kernel when the shape allows it and the CUDA-core fp32 kernel otherwise.
 * ---------------------------------------------------------------------- */
#define KIVI_ATTN_AUTO 0
#define KIVI_ATTN_FP32 1 /* CUDA-core fp32 kernel, any supported shape */
#define KIVI_ATTN_MMA 2  /* tensor-core kernel: D=128, G=32, n_rep<=8, bf16 or f32 q */

size_t kivi_decode_attention_workspace(int num_units, int n_rep, int head_dim, int num_splits);
int kivi_decode_attention_max_splits(void);

/* The plan kivi_decode_attention follows for a problem of this shape (host
 * arithmetic only, nothing is launched): whether the tensor-core kernel runs,
 * into how many pieces every unit's quantized history is cut (num_splits > 0 is
 * taken as given, 0 lets the library choose from the number of CTAs the GPU
 * holds at a time) and how many CTAs per unit take the residual ring.
 * sms / ctas_per_sm: the SM count and the tensor-core kernel's resident CTAs per
 * SM to plan for; <= 0 asks the current device (148 and 3 without one).
 * No counterpart in the reference. */
int kivi_decode_attention_plan(int num_units, int64_t quant_len, int res_len, int head_dim, int group_size,
                               int n_rep, int q_dtype, int num_splits, int path, int sms, int ctas_per_sm,
                               int* tensor_cores_out, int* quant_splits_out, int* residual_parts_out);

int kivi_decode_attention(const kivi_layer* layer, int64_t quant_len, int res_start,
                          int res_len, const void* q, int q_dtype, void* out, int out_dtype,
                          int n_rep, float sm_scale, void* workspace, size_t workspace_bytes,
                          int num_splits, int path, void* stream);

/* Same as kivi_decode_attention, and also writes lse_out[num_units][n_rep]
 * (fp32): the natural logarithm of the sum over all attended tokens of
 * exp(q.k * sm_scale).  With it, outputs computed over disjoint token ranges of
 * one sequence (a history sharded across GPUs, or a cache attended in pieces)
 * combine exactly: out = sum_i out_i * exp(lse_i - LSE), LSE = log sum_i exp(lse_i).
 * No counterpart in the reference.  The cache must hold at least one token. */
int kivi_decode_attention_lse(const kivi_layer* layer, int64_t quant_len, int res_start,
                              int res_len, const void* q, int q_dtype, void* out, int out_dtype,
                              float* lse_out, int n_rep, float sm_scale, void* workspace,
                              size_t workspace_bytes, int num_splits, int path, void* stream);

/* Folds attention results computed over disjoint token ranges of the same
 * sequences (a history sharded over GPUs by token groups): parts is device
 * [n_shards][rows][head_dim + 1] fp32, a row = the shard's output followed by its
 * log-sum-exp as written by kivi_decode_attention_lse (-inf for a shard that
 * held no token of the row).  out: device [rows][head_dim] of out_dtype;
 * lse_out (optional): the combined log-sum-exp.  No counterpart in the reference. */
int kivi_merge_token_shards(const float* parts, int n_shards, int64_t rows, int head_dim, void* out,
                            int out_dtype, float* lse_out, void* stream);

/* Decode attention for callers that cannot allocate device memory.
 *
 * No counterpart in the reference.  Some hosts of this library may not call
 * cudaMalloc at all: an inference server that hands every byte of HBM to its own
 * pool at start-up, a plug-in that runs inside another framework's memory plan,
 * a latency-critical loop where an allocation (which may synchronise the
 * device) is forbidden.  kivi_decode_attention needs a workspace from its
 * caller; this variant needs none.  Its split partials live in a fixed array
 * inside the library image (KIVI_NOALLOC_SCRATCH_BYTES, present on every GPU
 * that loads the library, for as long as the process lives), and the call
 * itself performs no cudaMalloc, cudaFree or any other allocating call.
 *
 * Same arguments and result as kivi_decode_attention minus the workspace.
 * Limit: num_units * (splits + residual parts) * n_rep * (head_dim + 2) * 4
 * bytes must fit in the array; a larger problem is refused with
 * KIVI_ERR_INVALID_ARGUMENT and a message naming the limit (pass a smaller
 * num_splits, or use kivi_decode_attention with your own workspace).
 * The first call on each device looks up the array's device address (no
 * allocation, but make that first call before starting a stream capture).
 * All calls on a device share the one array and nothing in it needs to start
 * at zero -- every slot that is read has been written by the same call -- but
 * two calls whose kernels overlap on the GPU (different streams, different
 * threads) would overwrite each other's partials: serialise them. */
#define KIVI_NOALLOC_SCRATCH_BYTES (8u << 20)
int kivi_decode_attention_noalloc(const kivi_layer* layer, int64_t quant_len, int res_start,
                                  int res_len, const void* q, int q_dtype, void* out, int out_dtype,
                                  int n_rep, float sm_scale, int num_splits, int path, void* stream);

/* ------------------------------------------------------------------------
 * Decode attention whose output goes straight into every GPU's gathered buffer.
 *
 * No counterpart in the reference (it is single-device).  With the (batch,
 * kv_head) units sharded over the GPUs of one node, the one exchange per
 * layer-step is an all-gather of the attention outputs.  Instead of a separate
 * collective, the kernel that folds the split partials writes each output row
 * into the gathered buffer of every rank through peer-mapped pointers (plain
 * stores over NVLink; no multicast, no TMA), publishes "rank r finished epoch e"
 * in every rank's flag array and, if asked, waits until all ranks have
 * published the same epoch -- so when the call's last kernel completes, this
 * rank's gathered buffer is complete.
 *
 * Buffers: kivi_peer_alloc makes a zeroed device allocation and its 64-byte
 * inter-process handle; every other rank maps it with kivi_peer_open (same
 * node, peer access over NVLink) and unmaps it with kivi_peer_close before the
 * owner calls kivi_peer_free.  Exchange the handles with any host-side channel.
 *
 * kivi_peer_gather: out_ptrs[r] = rank r's gathered buffer
 * [total_units][n_rep][D] of out_dtype as addressable from this GPU (own
 * allocation for r == rank), flag_ptrs[r] = rank r's uint32[world] flag array
 * (zero before the first call), unit_offset = index of this rank's first unit
 * in the gathered buffer, epoch = 1, 2, 3, ... identical on all ranks per call.
 * wait != 0: bounded wait for all ranks (spin_limit polls of about 200 ns, 0 =
 * about a second); if it runs out the kernel returns, bit 1 of the device fault
 * word is set and the rows of the ranks that did not arrive are stale -- read
 * kivi_device_fault at the next point where the host synchronises anyway.
 * Re-use: a rank may run one call ahead of its peers, so alternate between two
 * gathered buffers (e.g. by epoch parity) when the consumer of call e may still
 * be reading while call e+1 of a faster rank writes.
 * epoch_dev != NULL (for a call captured in a CUDA graph, whose arguments are
 * frozen): the epoch is kept on the device.  The call's epoch is *epoch_dev + 1,
 * which the kernel stores back when it is done; `epoch` is ignored; out_ptrs[r]
 * names the first of rank r's two gathered buffers, alt_bytes apart, and the
 * call writes buffer (epoch & 1).  Every rank keeps its own counter (zero before
 * the first call); all ranks must make the same sequence of calls.
 * ---------------------------------------------------------------------- */
#define KIVI_PEER_MAX_WORLD 8
typedef struct kivi_peer_gather {
    int rank, world;
    void* out_ptrs[KIVI_PEER_MAX_WORLD];
    uint32_t* flag_ptrs[KIVI_PEER_MAX_WORLD];
    int64_t unit_offset;
    uint32_t epoch;
    int wait;
    uint32_t spin_limit; /* polls (about 200 ns each) the wait may take; 0 = about a second */
    uint32_t reserved;
    uint64_t* wait_stats; /* optional device uint64[2]: the kernel adds the nanoseconds it spent waiting
                             for the other ranks to [0] and 1 to [1]; NULL = not recorded */
    uint32_t* epoch_dev;  /* optional device counter of this rank's calls (see above); NULL = use `epoch` */
    int64_t alt_bytes;    /* with epoch_dev: distance in bytes between a rank's two gathered buffers */
} kivi_peer_gather;

int kivi_peer_alloc(size_t bytes, void** ptr_out, unsigned char handle_out[64]);
int kivi_peer_open(const unsigned char handle[64], void** ptr_out);
int kivi_peer_close(void* ptr);
int kivi_peer_free(void* ptr);

int kivi_decode_attention_gather(const kivi_layer* layer, int64_t quant_len, int res_start,
                                 int res_len, const void* q, int q_dtype,
                                 const kivi_peer_gather* gather, int out_dtype,
                                 int n_rep, float sm_scale, void* workspace, size_t workspace_bytes,
                                 int num_splits, int path, void* stream);

/* Reads (and synchronises with) the device fault word: bit 0 is set once a wait
 * for a bulk copy inside a kernel of this library ran out, bit 1 once a wait for
 * peer ranks in kivi_decode_attention_gather ran out.  Such a kernel returns
 * normally (bit 0: the affected split counts as empty).  The word is sticky
 * until kivi_device_fault_clear() resets it (current device; synchronises). */
int kivi_device_fault(int* word_out);
int kivi_device_fault_clear(void);

/* ------------------------------------------------------------------------
 * One decode layer-step from and to pinned host memory.
 *
 * replaces the cache side of one iteration of the reference's decode loop --
 * add_tokens() of the step's new token, then serving the cache to the attention
 * (generation/generate.py:72-77, cache/manager.py:162-290) -- for a host that
 * holds q and the new K/V token in pinned memory and wants the attention output
 * back there.  In stream order on `stream`: copy in, kivi_cache_update with one
 * new token per unit (counters are read from and written back to *quant_len,
 * *res_start, *res_len), kivi_decode_attention, copy out.  Nothing is
 * synchronised: wait for `stream` before reading h_out.
 * h_q, h_out: [num_units][n_rep][D]; h_new_k, h_new_v: [num_units][D]; dtype
 * applies to q / new K / new V, out_dtype to h_out.
 * direct != 0: the kernels read and write the pinned host buffers themselves
 * (no copy operation; d_stage may be NULL).  direct == 0: explicit copies through
 * d_stage, device scratch of kivi_decode_step_stage_bytes(); chunks (1..4) then
 * cuts the units into that many runs handled on separate streams of the library,
 * so one run's copies overlap another's kernels; every run gets its share of
 * `workspace` (kivi_decode_attention_workspace of the whole layer is enough).
 * gather != NULL: the attention is kivi_decode_attention_gather (chunks = 1) and
 * h_out receives the first gather_units rows of this rank's gathered buffer.
 * ---------------------------------------------------------------------- */
size_t kivi_decode_step_stage_bytes(int num_units, int n_rep, int head_dim);
int kivi_decode_step_host(const kivi_layer* layer, int64_t* quant_len, int* res_start, int* res_len,
                          const void* h_q, const void* h_new_k, const void* h_new_v, void* h_out,
                          int dtype, int out_dtype, int n_rep, float sm_scale,
                          void* d_stage, size_t d_stage_bytes, void* workspace, size_t workspace_bytes,
                          int num_splits, int path, int rounding, int chunks, int direct,
                          const kivi_peer_gather* gather, int64_t gather_units, void* stream);

/* ------------------------------------------------------------------------
 * Next-token choice on the device.
 *
 * replaces sample_token, src/kivi_sycl/generation/sampling.py:10-25 (torch on
 * the host there): ids_out[b] = argmax of row b, or with do_sample != 0 one draw
 * from softmax(logits / max(temperature, 1e-8)) restricted to the entries not
 * below the top_k-th largest (top_k = 0: no cut; ties with the k-th are kept).
 * logits: device [batch][row_stride >= vocab] of dtype; ids_out: device int64[batch].
 * The draw of row b is the inverse CDF, in index order, at the uniform number
 * (w + 0.5) / 2^32, w = first output word of Philox4x32-10 with key `seed` and
 * counter (step, b): the same (seed, step) gives the same ids, and a host
 * restatement can reproduce them.  Ties of the argmax go to the lowest index.
 * ---------------------------------------------------------------------- */
int kivi_sample_tokens(const void* logits, int dtype, int batch, int vocab, int64_t row_stride,
                       float temperature, int top_k, int do_sample, uint64_t seed, uint64_t step,
                       int64_t* ids_out, void* stream);

/* Self-test (allocates 4 bytes, synchronises): the largest k for which the
 * tensor core, adding the products 1 and 2^-k to the addend -1 in one m16n8k16
 * fp16 MMA, still returns exactly 2^-k -- i.e. how many bits below the largest
 * addend survive its alignment (25 on B200).  The tensor-core attention kernel
 * feeds 2-bit codes as fp16 subnormals and places them so that at least 20 of
 * those bits are left for every code; below 24 here its error bound does not
 * hold.  No counterpart in the reference. */
int kivi_selftest_mma_alignment_bits(int* bits_out);

/* number of kernels the last successful call on this thread launched */
int kivi_last_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* KIVI_CUDA_H_ */
