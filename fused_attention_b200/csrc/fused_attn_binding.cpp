// Torch extension module `fused_attn`: the operator surface of the reference binding
// (src/fused_attn_extention.cu:15-129) over the C ABI of include/fa_b200.h.
//
//   fused_attn.attention_forward(head_dim, chunk_size, queries, keys, values, mask=None) -> Tensor
//
// Same argument names, order and default; the same preconditions raise the same exception type
// (c10::Error -> RuntimeError).  Relaxed on purpose: sequence_len need not be a multiple of
// chunk_size.  Fixed on purpose: the output lives on queries.device() and the launch goes to the
// caller's current stream (the reference allocates on the current device and launches on stream 0,
// src/fused_attn_extention.cu:67-70, include/fused_attn.cuh:885).
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "fa_b200.h"

namespace {

void check_input(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.dtype() == torch::kFloat16 && t.device().type() == torch::kCUDA && t.is_contiguous() &&
                    t.dim() == 3,
                name, " must be a contiguous float16 CUDA tensor with 3 dimensions");
}

torch::Tensor attention_forward(int head_dim, int chunk_size, torch::Tensor queries, torch::Tensor keys,
                                torch::Tensor values, torch::optional<torch::Tensor> mask) {
    check_input(queries, "queries");
    check_input(keys, "keys");
    check_input(values, "values");
    if (mask.has_value()) check_input(*mask, "mask");

    TORCH_CHECK(head_dim > 0 && !(head_dim & (head_dim - 1)) && 16 <= head_dim && head_dim <= 128,
                "head_dim must be a power of two in [16, 128]");
    TORCH_CHECK(chunk_size > 0 && !(chunk_size & (chunk_size - 1)) && 16 <= chunk_size && chunk_size <= 128 &&
                    chunk_size <= 2 * head_dim,
                "chunk_size must be a power of two in [16, 128] and at most 2*head_dim");
    TORCH_CHECK(!(chunk_size == 16 && head_dim == 128), "chunk_size 16 with head_dim 128 is not supported");

    const int64_t B = queries.size(0), L = queries.size(1), F = queries.size(2);
    TORCH_CHECK(keys.size(0) == B && keys.size(1) == L && keys.size(2) == F, "keys must have the shape of queries");
    TORCH_CHECK(values.size(0) == B && values.size(1) == L && values.size(2) == F,
                "values must have the shape of queries");
    TORCH_CHECK(F % head_dim == 0, "the feature size must be divisible by head_dim");
    TORCH_CHECK(B > 0 && L > 0 && F > 0, "empty tensors are not supported");
    TORCH_CHECK(keys.device() == queries.device() && values.device() == queries.device(),
                "queries, keys and values must be on one device");
    if (mask.has_value()) {
        TORCH_CHECK(mask->size(0) == B && mask->size(1) == L && mask->size(2) == L, "mask must have shape [B, L, L]");
        TORCH_CHECK(mask->device() == queries.device(), "mask must be on the device of queries");
    }

    const c10::cuda::CUDAGuard guard(queries.device());
    auto output = torch::empty_like(queries);
    const auto stream = c10::cuda::getCurrentCUDAStream(queries.device().index());
    const int rc = fa_b200_attention_forward(
        queries.data_ptr(), keys.data_ptr(), values.data_ptr(), mask.has_value() ? mask->data_ptr() : nullptr,
        output.data_ptr(), static_cast<uint32_t>(B), static_cast<uint32_t>(L), static_cast<uint32_t>(F),
        static_cast<uint32_t>(head_dim), static_cast<uint32_t>(chunk_size), queries.device().index(),
        static_cast<void*>(stream.stream()), FA_B200_FLAG_DEFAULT);
    TORCH_CHECK(rc == FA_B200_OK, "fa_b200: ", fa_b200_strerror(rc), " (status ", rc, ")");
    return output;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("attention_forward", &attention_forward, py::arg("head_dim"), py::arg("chunk_size"), py::arg("queries"),
          py::arg("keys"), py::arg("values"), py::arg("mask") = torch::optional<torch::Tensor>(),
          "Fused multihead attention");
}
