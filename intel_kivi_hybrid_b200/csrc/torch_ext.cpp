// kivi_cuda._C: the torch extension that mirrors the reference's pybind module
// (src/csrc/bindings/pybind_module.cpp:9-82) over libkivi_cuda's C ABI.
//
// Same twelve operators with the same positional and keyword names, the same
// caller-allocates-everything contract and the same argument checks as the
// reference's validate_* helpers (src/csrc/ops/kv_cache_ops.cpp:19-171), raised
// as RuntimeError before anything is launched.  Differences, all additive:
// tensors live on a CUDA device, `input` of the quantize / round-trip operators
// may be bfloat16 as well as float32, kernels are enqueued on torch's current
// CUDA stream (the counterpart of kivi::get_queue, include/kivi/common.hpp:26),
// and an optional `rounding` keyword selects half-even rounding.
//
// Blocking operators return after the kernel has finished, like the reference's
// wait_and_throw (quantize_kernels.cpp:64-66); *_async operators return a
// KiviEvent recorded behind the kernel (event.hpp:18-29).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kivi_cuda.h"

namespace {

void check_tensor(const torch::Tensor& t, const char* name, torch::ScalarType expected) {
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.scalar_type() == expected, name, " must be ", torch::toString(expected), " but got ",
                torch::toString(t.scalar_type()));
    TORCH_CHECK(t.is_cuda(), name, " must be on cuda but got ", t.device().str());
}

// Every operand of one operator must live on the same GPU: the kernel runs on
// the first operand's device and would otherwise dereference another GPU's
// pointers.  Checked before anything is launched.
void check_same_device(const torch::Tensor& first, const char* first_name, const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.device() == first.device(), name, " is on ", t.device().str(), " but ", first_name, " is on ",
                first.device().str(), ": all tensors of one call must be on the same device");
}

// input of quantize / round trip: float32 (reference) or bfloat16 (extension)
int check_input(const torch::Tensor& t) {
    TORCH_CHECK(t.is_contiguous(), "input must be contiguous");
    TORCH_CHECK(t.scalar_type() == torch::kFloat32 || t.scalar_type() == torch::kBFloat16,
                "input must be Float or BFloat16 but got ", torch::toString(t.scalar_type()));
    TORCH_CHECK(t.is_cuda(), "input must be on cuda but got ", t.device().str());
    return t.scalar_type() == torch::kFloat32 ? KIVI_F32 : KIVI_BF16;
}

void check(int rc) { TORCH_CHECK(rc == KIVI_OK, "kivi_cuda: ", kivi_last_error()); }

void* stream_of(const torch::Tensor& t) {
    return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

struct KiviEvent {
    cudaEvent_t ev = nullptr;
    explicit KiviEvent(void* stream) {
        C10_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        C10_CUDA_CHECK(cudaEventRecord(ev, (cudaStream_t)stream));
    }
    KiviEvent(const KiviEvent&) = delete;
    KiviEvent(KiviEvent&& o) noexcept : ev(o.ev) { o.ev = nullptr; }
    ~KiviEvent() { if (ev) cudaEventDestroy(ev); }
    void wait() { C10_CUDA_CHECK(cudaEventSynchronize(ev)); }
};

int64_t validate_quant_keys(const torch::Tensor& input, const torch::Tensor& output, const torch::Tensor& scales,
                            const torch::Tensor& zeros, int group_size) {
    check_input(input);
    check_tensor(output, "output", torch::kUInt8);
    check_tensor(scales, "scales", torch::kFloat32);
    check_tensor(zeros, "zeros", torch::kFloat32);
    check_same_device(input, "input", output, "output");
    check_same_device(input, "input", scales, "scales");
    check_same_device(input, "input", zeros, "zeros");
    TORCH_CHECK(group_size > 0 && group_size % 4 == 0, "group_size must be positive and divisible by 4, got ", group_size);
    const int64_t n = scales.numel();
    TORCH_CHECK(n > 0, "scales must be non-empty");
    TORCH_CHECK(zeros.numel() == n, "zeros size (", zeros.numel(), ") must match scales size (", n, ")");
    TORCH_CHECK(input.numel() == n * group_size, "input size (", input.numel(), ") must equal num_channels(", n,
                ") * group_size(", group_size, ") = ", n * group_size);
    TORCH_CHECK(output.numel() == n * (group_size / 4), "output size (", output.numel(), ") must equal num_channels(", n,
                ") * (group_size/4) = ", n * (group_size / 4));
    return n;
}

int64_t validate_quant_values(const torch::Tensor& input, const torch::Tensor& output, const torch::Tensor& scales,
                              const torch::Tensor& zeros, int head_dim, int group_size) {
    check_input(input);
    check_tensor(output, "output", torch::kUInt8);
    check_tensor(scales, "scales", torch::kFloat32);
    check_tensor(zeros, "zeros", torch::kFloat32);
    check_same_device(input, "input", output, "output");
    check_same_device(input, "input", scales, "scales");
    check_same_device(input, "input", zeros, "zeros");
    TORCH_CHECK(group_size > 0 && group_size % 4 == 0, "group_size must be positive and divisible by 4");
    TORCH_CHECK(head_dim > 0 && head_dim % group_size == 0, "head_dim must be positive and divisible by group_size");
    TORCH_CHECK(input.numel() % head_dim == 0, "input.numel() (", input.numel(), ") must be divisible by head_dim (",
                head_dim, ") - refusing to silently truncate trailing elements");
    const int64_t tokens = input.numel() / head_dim, gpt = head_dim / group_size;
    TORCH_CHECK(tokens > 0, "input must be non-empty");
    TORCH_CHECK(scales.numel() == tokens * gpt, "scales size (", scales.numel(), ") must equal num_tokens(", tokens,
                ") * groups_per_token(", gpt, ")");
    TORCH_CHECK(zeros.numel() == scales.numel(), "zeros size (", zeros.numel(), ") must match scales size (", scales.numel(), ")");
    TORCH_CHECK(output.numel() == tokens * (head_dim / 4), "output size (", output.numel(), ") must equal num_tokens(",
                tokens, ") * (head_dim/4) = ", tokens * (head_dim / 4));
    return tokens;
}

int64_t validate_dequant(const torch::Tensor& input, const torch::Tensor& scales, const torch::Tensor& zeros,
                         const torch::Tensor& output, int group_size, const char* what) {
    check_tensor(input, "input", torch::kUInt8);
    check_tensor(scales, "scales", torch::kFloat32);
    check_tensor(zeros, "zeros", torch::kFloat32);
    check_tensor(output, "output", torch::kFloat32);
    check_same_device(input, "input", scales, "scales");
    check_same_device(input, "input", zeros, "zeros");
    check_same_device(input, "input", output, "output");
    TORCH_CHECK(group_size > 0 && group_size % 4 == 0, "group_size must be positive and divisible by 4, got ", group_size);
    const int64_t n = scales.numel();
    TORCH_CHECK(n > 0, "scales must be non-empty");
    TORCH_CHECK(zeros.numel() == n, "zeros size (", zeros.numel(), ") must match scales size (", n, ")");
    TORCH_CHECK(input.numel() == n * (group_size / 4), "input (packed) size (", input.numel(), ") must equal ", what, "(", n,
                ") * (group_size/4) = ", n * (group_size / 4));
    TORCH_CHECK(output.numel() == n * group_size, "output size (", output.numel(), ") must equal ", what, "(", n,
                ") * group_size = ", n * group_size);
    return n;
}

int64_t validate_roundtrip_keys(const torch::Tensor& input, const torch::Tensor& output, int group_size) {
    check_input(input);
    check_tensor(output, "output", torch::kFloat32);
    check_same_device(input, "input", output, "output");
    TORCH_CHECK(group_size > 0 && group_size % 4 == 0, "group_size must be positive and divisible by 4, got ", group_size);
    TORCH_CHECK(input.numel() % group_size == 0, "input.numel() (", input.numel(), ") must be divisible by group_size (", group_size, ")");
    TORCH_CHECK(output.numel() == input.numel(), "output size (", output.numel(), ") must equal input size (", input.numel(),
                ") - round-trip is shape-preserving");
    const int64_t n = input.numel() / group_size;
    TORCH_CHECK(n > 0, "input must be non-empty");
    return n;
}

int64_t validate_roundtrip_values(const torch::Tensor& input, const torch::Tensor& output, int head_dim, int group_size) {
    check_input(input);
    check_tensor(output, "output", torch::kFloat32);
    check_same_device(input, "input", output, "output");
    TORCH_CHECK(group_size > 0 && group_size % 4 == 0, "group_size must be positive and divisible by 4");
    TORCH_CHECK(head_dim > 0 && head_dim % group_size == 0, "head_dim must be positive and divisible by group_size");
    TORCH_CHECK(input.numel() % head_dim == 0, "input.numel() (", input.numel(), ") must be divisible by head_dim (", head_dim, ")");
    TORCH_CHECK(output.numel() == input.numel(), "output size (", output.numel(), ") must equal input size (", input.numel(),
                ") - round-trip is shape-preserving");
    const int64_t n = input.numel() / head_dim;
    TORCH_CHECK(n > 0, "input must be non-empty");
    return n;
}

int dtype_code(const torch::Tensor& t) { return t.scalar_type() == torch::kFloat32 ? KIVI_F32 : KIVI_BF16; }

// ---- enqueue helpers (shared by the blocking and the _async twins) -----------
void* enqueue_quant_keys(torch::Tensor& input, torch::Tensor& output, torch::Tensor& scales, torch::Tensor& zeros,
                         int group_size, int rounding) {
    const int64_t n = validate_quant_keys(input, output, scales, zeros, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    void* st = stream_of(input);
    check(kivi_quantize_keys_per_channel(input.data_ptr(), dtype_code(input), output.data_ptr<uint8_t>(),
                                         scales.data_ptr<float>(), zeros.data_ptr<float>(), n, group_size, rounding, st));
    return st;
}
void* enqueue_quant_values(torch::Tensor& input, torch::Tensor& output, torch::Tensor& scales, torch::Tensor& zeros,
                           int head_dim, int group_size, int rounding) {
    const int64_t n = validate_quant_values(input, output, scales, zeros, head_dim, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    void* st = stream_of(input);
    check(kivi_quantize_values_per_token(input.data_ptr(), dtype_code(input), output.data_ptr<uint8_t>(),
                                         scales.data_ptr<float>(), zeros.data_ptr<float>(), n, head_dim, group_size, rounding, st));
    return st;
}
void* enqueue_dequant_keys(torch::Tensor& input, torch::Tensor& scales, torch::Tensor& zeros, torch::Tensor& output, int group_size) {
    const int64_t n = validate_dequant(input, scales, zeros, output, group_size, "num_channels");
    c10::cuda::CUDAGuard guard(input.device());
    void* st = stream_of(input);
    check(kivi_dequantize_keys_per_channel(input.data_ptr<uint8_t>(), scales.data_ptr<float>(), zeros.data_ptr<float>(),
                                           output.data_ptr<float>(), n, group_size, st));
    return st;
}
void* enqueue_dequant_values(torch::Tensor& input, torch::Tensor& scales, torch::Tensor& zeros, torch::Tensor& output,
                             int head_dim, int group_size) {
    TORCH_CHECK(head_dim > 0 && group_size > 0 && head_dim % group_size == 0, "head_dim must be positive and divisible by group_size");
    const int64_t n = validate_dequant(input, scales, zeros, output, group_size, "num_groups");
    c10::cuda::CUDAGuard guard(input.device());
    void* st = stream_of(input);
    check(kivi_dequantize_values_per_token(input.data_ptr<uint8_t>(), scales.data_ptr<float>(), zeros.data_ptr<float>(),
                                           output.data_ptr<float>(), n, group_size, st));
    return st;
}
void* enqueue_roundtrip_keys(torch::Tensor& input, torch::Tensor& output, int group_size, int rounding) {
    const int64_t n = validate_roundtrip_keys(input, output, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    void* st = stream_of(input);
    check(kivi_quant_dequant_roundtrip_keys(input.data_ptr(), dtype_code(input), output.data_ptr<float>(), n, group_size, rounding, st));
    return st;
}
void* enqueue_roundtrip_values(torch::Tensor& input, torch::Tensor& output, int head_dim, int group_size, int rounding) {
    const int64_t n = validate_roundtrip_values(input, output, head_dim, group_size);
    c10::cuda::CUDAGuard guard(input.device());
    void* st = stream_of(input);
    check(kivi_quant_dequant_roundtrip_values(input.data_ptr(), dtype_code(input), output.data_ptr<float>(), n, head_dim,
                                              group_size, rounding, st));
    return st;
}

// the blocking operators wait with the GIL released, so other Python threads run
// while the kernel does (the reference holds it, bindings/pybind_module.cpp:18-49)
void block_on(void* st) {
    cudaError_t e;
    {
        py::gil_scoped_release nogil;
        e = cudaStreamSynchronize((cudaStream_t)st);
    }
    C10_CUDA_CHECK(e);
}



// ---- the cache operators (no counterpart in the reference's module: there the
// cache is Python over round-trip kernels, cache/manager.py:162-374) -------------
// The packed store of one layer as tensors the caller owns:
//   k_packed [units, max_groups, D*G/4] u8, k_scales / k_zeros [units, max_groups, D] f32,
//   v_packed [units, max_tokens, D/4] u8,   v_scales / v_zeros [units, max_tokens, D/G] f32,
//   k_res / v_res [units, R, D] f32 or bf16 (the residual ring),
// with max_tokens = max_groups * G.  Only dtypes, devices, contiguity and numel
// relations are checked, like the reference's validators.
kivi_layer layer_of(const torch::Tensor& k_packed, const torch::Tensor& k_scales, const torch::Tensor& k_zeros,
                    const torch::Tensor& v_packed, const torch::Tensor& v_scales, const torch::Tensor& v_zeros,
                    const torch::Tensor& k_res, const torch::Tensor& v_res, int group_size) {
    check_tensor(k_packed, "k_packed", torch::kUInt8);
    check_tensor(v_packed, "v_packed", torch::kUInt8);
    check_tensor(k_scales, "k_scales", torch::kFloat32);
    check_tensor(k_zeros, "k_zeros", torch::kFloat32);
    check_tensor(v_scales, "v_scales", torch::kFloat32);
    check_tensor(v_zeros, "v_zeros", torch::kFloat32);
    TORCH_CHECK(k_res.dim() == 3 && v_res.sizes() == k_res.sizes(), "k_res and v_res must both be [units, R, D]");
    TORCH_CHECK(k_res.scalar_type() == torch::kFloat32 || k_res.scalar_type() == torch::kBFloat16,
                "k_res must be Float or BFloat16 but got ", torch::toString(k_res.scalar_type()));
    check_tensor(k_res, "k_res", k_res.scalar_type());
    check_tensor(v_res, "v_res", k_res.scalar_type());
    check_same_device(k_res, "k_res", v_res, "v_res");
    check_same_device(k_res, "k_res", k_packed, "k_packed");
    check_same_device(k_res, "k_res", k_scales, "k_scales");
    check_same_device(k_res, "k_res", k_zeros, "k_zeros");
    check_same_device(k_res, "k_res", v_packed, "v_packed");
    check_same_device(k_res, "k_res", v_scales, "v_scales");
    check_same_device(k_res, "k_res", v_zeros, "v_zeros");
    const int64_t units = k_res.size(0), R = k_res.size(1), D = k_res.size(2);
    const int G = group_size;
    TORCH_CHECK(G > 0 && G % 4 == 0, "group_size must be positive and divisible by 4, got ", G);
    TORCH_CHECK(D > 0 && D % G == 0, "head_dim (", D, ") must be divisible by group_size (", G, ")");
    TORCH_CHECK(units > 0 && k_scales.numel() % (units * D) == 0, "k_scales size (", k_scales.numel(),
                ") must be units(", units, ") * max_groups * head_dim(", D, ")");
    const int64_t max_groups = k_scales.numel() / (units * D), max_tokens = max_groups * G;
    TORCH_CHECK(k_zeros.numel() == k_scales.numel(), "k_zeros size must match k_scales size");
    TORCH_CHECK(k_packed.numel() == units * max_groups * (D * G / 4), "k_packed size (", k_packed.numel(),
                ") must equal units * max_groups * head_dim * group_size / 4 = ", units * max_groups * (D * G / 4));
    TORCH_CHECK(v_packed.numel() == units * max_tokens * (D / 4), "v_packed size (", v_packed.numel(),
                ") must equal units * max_tokens * head_dim / 4 = ", units * max_tokens * (D / 4));
    TORCH_CHECK(v_scales.numel() == units * max_tokens * (D / G) && v_zeros.numel() == v_scales.numel(),
                "v_scales / v_zeros size must equal units * max_tokens * head_dim / group_size = ", units * max_tokens * (D / G));
    kivi_layer L;
    L.num_units = (int32_t)units; L.head_dim = (int32_t)D; L.group_size = G; L.residual_cap = (int32_t)R;
    L.max_tokens = max_tokens; L.res_dtype = k_res.scalar_type() == torch::kFloat32 ? KIVI_F32 : KIVI_BF16; L.reserved = 0;
    L.k_codes = k_packed.data_ptr<uint8_t>(); L.k_scales = k_scales.data_ptr<float>(); L.k_zeros = k_zeros.data_ptr<float>();
    L.v_codes = v_packed.data_ptr<uint8_t>(); L.v_scales = v_scales.data_ptr<float>(); L.v_zeros = v_zeros.data_ptr<float>();
    L.k_res = k_res.data_ptr(); L.v_res = v_res.data_ptr();
    return L;
}

int dtype_code(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.scalar_type() == torch::kFloat32 || t.scalar_type() == torch::kBFloat16, name,
                " must be Float or BFloat16 but got ", torch::toString(t.scalar_type()));
    TORCH_CHECK(t.is_cuda(), name, " must be on cuda but got ", t.device().str());
    return t.scalar_type() == torch::kFloat32 ? KIVI_F32 : KIVI_BF16;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "KIVI: asymmetric 2-bit KV-cache quantization for NVIDIA B200 (sm_100a CUDA kernels)";
    m.attr("ROUND_HALF_AWAY") = KIVI_ROUND_HALF_AWAY;
    m.attr("ROUND_HALF_EVEN") = KIVI_ROUND_HALF_EVEN;

    py::class_<KiviEvent>(m, "KiviEvent",
        "Handle for a kernel submitted via a *_async op. Call .wait() before reading any tensor the kernel writes.")
        .def("wait", &KiviEvent::wait, py::call_guard<py::gil_scoped_release>(),
             "Block until the kernel completes; raises on a CUDA error.");

    using T = torch::Tensor;
    const int R0 = KIVI_ROUND_HALF_AWAY;
    m.def("quantize_keys", [](T input, T output, T scales, T zeros, int group_size, int rounding) {
              block_on(enqueue_quant_keys(input, output, scales, zeros, group_size, rounding)); },
          "Asymmetric 2-bit key quantization (per-channel)",
          py::arg("input"), py::arg("output"), py::arg("scales"), py::arg("zeros"), py::arg("group_size"), py::arg("rounding") = R0);
    m.def("quantize_values", [](T input, T output, T scales, T zeros, int head_dim, int group_size, int rounding) {
              block_on(enqueue_quant_values(input, output, scales, zeros, head_dim, group_size, rounding)); },
          "Asymmetric 2-bit value quantization (per-token)",
          py::arg("input"), py::arg("output"), py::arg("scales"), py::arg("zeros"), py::arg("head_dim"), py::arg("group_size"),
          py::arg("rounding") = R0);
    m.def("dequantize_keys", [](T input, T scales, T zeros, T output, int group_size) {
              block_on(enqueue_dequant_keys(input, scales, zeros, output, group_size)); },
          "Asymmetric 2-bit key dequantization (per-channel)",
          py::arg("input"), py::arg("scales"), py::arg("zeros"), py::arg("output"), py::arg("group_size"));
    m.def("dequantize_values", [](T input, T scales, T zeros, T output, int head_dim, int group_size) {
              block_on(enqueue_dequant_values(input, scales, zeros, output, head_dim, group_size)); },
          "Asymmetric 2-bit value dequantization (per-token)",
          py::arg("input"), py::arg("scales"), py::arg("zeros"), py::arg("output"), py::arg("head_dim"), py::arg("group_size"));
    m.def("quant_dequant_roundtrip_keys", [](T input, T output, int group_size, int rounding) {
              block_on(enqueue_roundtrip_keys(input, output, group_size, rounding)); },
          "Fused quantize->dequantize round-trip (per-channel); never writes packed bytes, scales or zeros.",
          py::arg("input"), py::arg("output"), py::arg("group_size"), py::arg("rounding") = R0);
    m.def("quant_dequant_roundtrip_values", [](T input, T output, int head_dim, int group_size, int rounding) {
              block_on(enqueue_roundtrip_values(input, output, head_dim, group_size, rounding)); },
          "Fused quantize->dequantize round-trip (per-token).",
          py::arg("input"), py::arg("output"), py::arg("head_dim"), py::arg("group_size"), py::arg("rounding") = R0);

    m.def("quantize_keys_async", [](T input, T output, T scales, T zeros, int group_size, int rounding) {
              return KiviEvent(enqueue_quant_keys(input, output, scales, zeros, group_size, rounding)); },
          "Non-blocking quantize_keys - returns a KiviEvent, does not wait.",
          py::arg("input"), py::arg("output"), py::arg("scales"), py::arg("zeros"), py::arg("group_size"), py::arg("rounding") = R0);
    m.def("quantize_values_async", [](T input, T output, T scales, T zeros, int head_dim, int group_size, int rounding) {
              return KiviEvent(enqueue_quant_values(input, output, scales, zeros, head_dim, group_size, rounding)); },
          "Non-blocking quantize_values - returns a KiviEvent, does not wait.",
          py::arg("input"), py::arg("output"), py::arg("scales"), py::arg("zeros"), py::arg("head_dim"), py::arg("group_size"),
          py::arg("rounding") = R0);
    m.def("dequantize_keys_async", [](T input, T scales, T zeros, T output, int group_size) {
              return KiviEvent(enqueue_dequant_keys(input, scales, zeros, output, group_size)); },
          "Non-blocking dequantize_keys - returns a KiviEvent, does not wait.",
          py::arg("input"), py::arg("scales"), py::arg("zeros"), py::arg("output"), py::arg("group_size"));
    m.def("dequantize_values_async", [](T input, T scales, T zeros, T output, int head_dim, int group_size) {
              return KiviEvent(enqueue_dequant_values(input, scales, zeros, output, head_dim, group_size)); },
          "Non-blocking dequantize_values - returns a KiviEvent, does not wait.",
          py::arg("input"), py::arg("scales"), py::arg("zeros"), py::arg("output"), py::arg("head_dim"), py::arg("group_size"));
    m.def("quant_dequant_roundtrip_keys_async", [](T input, T output, int group_size, int rounding) {
              return KiviEvent(enqueue_roundtrip_keys(input, output, group_size, rounding)); },
          "Non-blocking quant_dequant_roundtrip_keys - returns a KiviEvent, does not wait.",
          py::arg("input"), py::arg("output"), py::arg("group_size"), py::arg("rounding") = R0);
    m.def("quant_dequant_roundtrip_values_async", [](T input, T output, int head_dim, int group_size, int rounding) {
              return KiviEvent(enqueue_roundtrip_values(input, output, head_dim, group_size, rounding)); },
          "Non-blocking quant_dequant_roundtrip_values - returns a KiviEvent, does not wait.",
          py::arg("input"), py::arg("output"), py::arg("head_dim"), py::arg("group_size"), py::arg("rounding") = R0);

    // ---- cache operators ---------------------------------------------------------
    m.def("append_and_flush",
          [](T new_k, T new_v, T k_packed, T k_scales, T k_zeros, T v_packed, T v_scales, T v_zeros, T k_res, T v_res,
             int64_t quant_len, int res_start, int res_len, int group_size, int rounding) {
              kivi_layer L = layer_of(k_packed, k_scales, k_zeros, v_packed, v_scales, v_zeros, k_res, v_res, group_size);
              const int dt = dtype_code(new_k, "new_k");
              TORCH_CHECK(new_v.scalar_type() == new_k.scalar_type() && new_v.is_cuda(), "new_v must match new_k's dtype and device");
              check_same_device(k_res, "k_res", new_k, "new_k");
              check_same_device(k_res, "k_res", new_v, "new_v");
              c10::cuda::CUDAGuard guard(k_res.device());
              TORCH_CHECK(new_k.dim() == 3 && new_k.sizes() == new_v.sizes() && new_k.size(0) == L.num_units && new_k.size(2) == L.head_dim,
                          "new_k / new_v must be [units, n_new, head_dim]");
              TORCH_CHECK(new_k.stride(2) == 1 && new_v.stride(2) == 1, "the last dimension of new_k / new_v must be contiguous");
              int64_t ql = 0; int rs = 0, rl = 0;
              check(kivi_cache_update(&L, quant_len, res_start, res_len, new_k.data_ptr(), new_v.data_ptr(), dt,
                                      new_k.stride(0), new_k.stride(1), new_v.stride(0), new_v.stride(1), (int)new_k.size(1),
                                      rounding, &ql, &rs, &rl, stream_of(k_res)));
              return std::make_tuple(ql, rs, rl);
          },
          "Append n_new tokens to a layer's cache: while the ring holds >= R tokens its oldest group_size tokens are "
          "quantized into the packed store (add_tokens + _flush_group of the reference, cache/manager.py:162-374), all on "
          "the device and in stream order.  Returns the new (quant_len, res_start, res_len).",
          py::arg("new_k"), py::arg("new_v"), py::arg("k_packed"), py::arg("k_scales"), py::arg("k_zeros"),
          py::arg("v_packed"), py::arg("v_scales"), py::arg("v_zeros"), py::arg("k_res"), py::arg("v_res"),
          py::arg("quant_len"), py::arg("res_start"), py::arg("res_len"), py::arg("group_size"), py::arg("rounding") = R0);
    m.def("decode_attention",
          [](T q, T k_packed, T k_scales, T k_zeros, T v_packed, T v_scales, T v_zeros, T k_res, T v_res,
             int64_t quant_len, int res_start, int res_len, T out, int group_size, c10::optional<T> workspace,
             double sm_scale, int num_splits, int path) {
              kivi_layer L = layer_of(k_packed, k_scales, k_zeros, v_packed, v_scales, v_zeros, k_res, v_res, group_size);
              const int qd = dtype_code(q, "q"), od = dtype_code(out, "out");
              check_same_device(k_res, "k_res", q, "q");
              check_same_device(k_res, "k_res", out, "out");
              if (workspace.has_value()) check_same_device(k_res, "k_res", *workspace, "workspace");
              c10::cuda::CUDAGuard guard(k_res.device());
              TORCH_CHECK(q.is_contiguous() && out.is_contiguous(), "q and out must be contiguous");
              TORCH_CHECK(q.numel() == out.numel() && q.numel() % ((int64_t)L.num_units * L.head_dim) == 0 && q.numel() > 0,
                          "q and out must both hold units * n_rep * head_dim elements");
              const int n_rep = (int)(q.numel() / ((int64_t)L.num_units * L.head_dim));
              const size_t need = kivi_decode_attention_workspace(L.num_units, n_rep, L.head_dim, num_splits);
              T ws = workspace.has_value() ? *workspace
                                           : torch::empty({(int64_t)need}, torch::TensorOptions().dtype(torch::kUInt8).device(k_res.device()));
              check_tensor(ws, "workspace", torch::kUInt8);
              check(kivi_decode_attention(&L, quant_len, res_start, res_len, q.data_ptr(), qd, out.data_ptr(), od, n_rep,
                                          (float)sm_scale, ws.data_ptr(), (size_t)ws.numel(), num_splits, path, stream_of(k_res)));
          },
          "Fused decode attention over a layer's packed cache: out = softmax(q K^T * sm_scale) V over [quantized history || "
          "residual ring] (the math of tests/integration/test_attention_fix.py:40-43), no dequantized cache is built.  "
          "q, out: [units, n_rep, head_dim]; stream-ordered; workspace: optional uint8 scratch "
          "(kivi_decode_attention_workspace bytes), allocated per call when omitted.",
          py::arg("q"), py::arg("k_packed"), py::arg("k_scales"), py::arg("k_zeros"), py::arg("v_packed"), py::arg("v_scales"),
          py::arg("v_zeros"), py::arg("k_res"), py::arg("v_res"), py::arg("quant_len"), py::arg("res_start"), py::arg("res_len"),
          py::arg("out"), py::arg("group_size"), py::arg("workspace") = py::none(), py::arg("sm_scale") = 0.0,
          py::arg("num_splits") = 0, py::arg("path") = 0);
    m.def("decode_attention_workspace", [](int num_units, int n_rep, int head_dim, int num_splits) {
              return (int64_t)kivi_decode_attention_workspace(num_units, n_rep, head_dim, num_splits); },
          "Bytes of scratch decode_attention needs.", py::arg("num_units"), py::arg("n_rep"), py::arg("head_dim"), py::arg("num_splits") = 0);
}
