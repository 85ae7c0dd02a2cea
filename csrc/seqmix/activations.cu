// Elementwise activations and the small-batch pieces of a routed feed-forward.
//   xielu        : z > 0: ap z^2 + z/2;  z <= 0: an (exp(z) - 1 - z) + z/2   (ap, an are positive numbers prepared by the caller)
//   gelu_erf     : 0.5 z (1 + erf(z / sqrt 2))
//   indexed_gemv : out[m,:] = act(W[sel[m]] x[m,:]) for a few rows m, each with its own matrix out of a stack [E, O, I]
//                  (token generation: the chosen experts' matrices are streamed once, a warp per output row)
//   moe_combine  : y[n,:] = base[n,:] + sum_k weight[n,k] * rows[src[n,k],:], summed in float
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

__device__ __forceinline__ float gelu_erf_(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752f)); }

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ x, T* __restrict__ out, long n, float ap, float an) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = ldf(x + i);
    stf(out + i, z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z));
}

template <typename T>
__global__ void gelu_erf_kernel(const T* __restrict__ x, T* __restrict__ out, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stf(out + i, gelu_erf_(ldf(x + i)));
}

template <typename T>
__global__ void indexed_gemv_kernel(const T* __restrict__ w, const int* __restrict__ sel, const T* __restrict__ x, long x_stride,
                                    int M, int O, int I, int act, T* __restrict__ out) {
    const int o = blockIdx.x * blockDim.y + threadIdx.y, m = blockIdx.y, lane = threadIdx.x;
    if (o >= O) return;
    const T* wr = w + ((long)sel[m] * O + o) * I;
    const T* xr = x + (long)m * x_stride;
    float acc = 0.f;
    for (int i = lane; i < I; i += 32) acc = fmaf(ldf(wr + i), ldf(xr + i), acc);
    acc = warp_sum(acc);
    if (lane == 0) stf(out + (long)m * O + o, act ? gelu_erf_(acc) : acc);
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ src, const float* __restrict__ weight,
                                   const T* __restrict__ base, int N, int top, int C, T* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, n = blockIdx.y;
    if (c >= C) return;
    float acc = base ? ldf(base + (long)n * C + c) : 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weight[(long)n * top + k], ldf(rows + (long)src[(long)n * top + k] * C + c), acc);
    stf(out + (long)n * C + c, acc);
}

void xielu(const void* x, void* out, int bf, long n, float ap, float an, cudaStream_t s) {
    if (n == 0) return;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (bf) xielu_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)x, (bf16*)out, n, ap, an);
    else xielu_kernel<float><<<blocks, 256, 0, s>>>((const float*)x, (float*)out, n, ap, an);
}

void gelu_erf(const void* x, void* out, int bf, long n, cudaStream_t s) {
    if (n == 0) return;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (bf) gelu_erf_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)x, (bf16*)out, n);
    else gelu_erf_kernel<float><<<blocks, 256, 0, s>>>((const float*)x, (float*)out, n);
}

void indexed_gemv(const void* w, const int* sel, const void* x, int bf, long x_stride, int M, int O, int I, int act, void* out,
                  cudaStream_t s) {
    if (M == 0) return;
    dim3 block(32, 8), grid((O + 7) / 8, M);
    if (bf) indexed_gemv_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)w, sel, (const bf16*)x, x_stride, M, O, I, act, (bf16*)out);
    else indexed_gemv_kernel<float><<<grid, block, 0, s>>>((const float*)w, sel, (const float*)x, x_stride, M, O, I, act, (float*)out);
}

void moe_combine(const void* rows, const int* src, const float* weight, const void* base, int bf, int N, int top, int C, void* out,
                 cudaStream_t s) {
    if (N == 0) return;
    dim3 block(128), grid((C + 127) / 128, N);
    if (bf) moe_combine_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)rows, src, weight, (const bf16*)base, N, top, C, (bf16*)out);
    else moe_combine_kernel<float><<<grid, block, 0, s>>>((const float*)rows, src, weight, (const float*)base, N, top, C, (float*)out);
}

}  // namespace seqmix
