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

void block_on(void* st) { C10_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)st)); }

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
}
