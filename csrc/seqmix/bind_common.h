// Helpers shared by the Python bindings of the sequence-mixer kernel groups: dtype / device / layout checks and the current stream.
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "seqmix.h"

using at::Tensor;

static int is_bf(const Tensor& t) {
    TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, "activations must be bfloat16 or float32");
    return t.scalar_type() == at::kBFloat16;
}
static const float* f32(const Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), "expected a contiguous float32 CUDA tensor");
    return t.data_ptr<float>();
}
static const int* i32(const Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), "expected a contiguous int32 CUDA tensor");
    return t.data_ptr<int>();
}
static cudaStream_t stream() { return at::cuda::getCurrentCUDAStream(); }
static void check_launch() {
    cudaError_t e = cudaGetLastError();
    TORCH_CHECK(e == cudaSuccess, "sequence-mixer kernel launch failed: ", cudaGetErrorString(e));
}

