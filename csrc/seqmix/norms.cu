// RMS norms of the sequence-mixer models: y = x / sqrt(mean(x^2) + eps) * w with w a vector or ONE number for all coordinates,
// optionally times silu(gate), written out or accumulated into a float residual stream (x_res += norm(y): the residual sum of a
// layer that normalises the sublayer's OUTPUT).  One warp per row; statistics in float.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

template <typename Tin, typename Tout>
__global__ void rms_norm_kernel(const Tin* __restrict__ x, long x_stride, int rows, int C, const float* __restrict__ w, int w_stride,
                                float eps, const Tout* __restrict__ gate, long gate_stride, Tout* __restrict__ out, long out_stride,
                                float* res, long res_stride) {
    const int row = blockIdx.x * blockDim.y + threadIdx.y, lane = threadIdx.x;
    if (row >= rows) return;
    const Tin* xr = x + (long)row * x_stride;
    float ss = 0.f;
    for (int c = lane; c < C; c += 32) { float v = ldf(xr + c); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)C + eps);
    for (int c = lane; c < C; c += 32) {
        float v = ldf(xr + c) * inv * w[(long)c * w_stride];
        if (gate) { float g = ldf(gate + (long)row * gate_stride + c); v *= g * sigmoidf_(g); }
        if (res) res[(long)row * res_stride + c] += v;
        else stf(out + (long)row * out_stride + c, v);
    }
}

void rms_norm(const void* x, int in_bf16, long x_stride, int rows, int C, const float* w, int w_stride, float eps, const void* gate,
              long gate_stride, void* out, int out_bf16, long out_stride, float* res, long res_stride, cudaStream_t s) {
    dim3 block(32, 8), grid((rows + 7) / 8);
#define SEQMIX_NORM(TI, TO)                                                                                                      \
    rms_norm_kernel<TI, TO><<<grid, block, 0, s>>>((const TI*)x, x_stride, rows, C, w, w_stride, eps, (const TO*)gate, gate_stride, \
                                                   (TO*)out, out_stride, res, res_stride)
    if (in_bf16 && out_bf16) SEQMIX_NORM(bf16, bf16);
    else if (!in_bf16 && out_bf16) SEQMIX_NORM(float, bf16);
    else if (!in_bf16 && !out_bf16) SEQMIX_NORM(float, float);
    else SEQMIX_NORM(bf16, float);
#undef SEQMIX_NORM
}

}  // namespace seqmix
