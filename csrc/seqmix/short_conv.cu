// Causal depthwise convolution over time with a carried history ("short convolution"): used as the residual input convolution of
// every sublayer (out = h + conv(h)) and as the plain convolution of the recurrent block (out = conv(h) + bias).
//   out[b,t,c] = sum_j w[c,j] * in(b, t - taps + 1 + j, c),   in(b,s,c) = x[b,s,c] for s >= 0, else the slot's history (zeros when
// the sequence starts in this call).  After the call the slot's history holds the last taps-1 inputs of the sequence (positions
// beyond lens[b] are padding: they produce zeros and never enter the history).
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kMaxTaps = 16;

template <typename Tin, typename Tout>
__global__ void short_conv_kernel(const Tin* __restrict__ x, long x_sb, long x_st, const float* __restrict__ w,
                                  const float* __restrict__ bias, Tin* state, const int* __restrict__ slots,
                                  const int* __restrict__ lens, int S, int C, int taps, int fresh, int residual,
                                  Tout* __restrict__ out) {
    const int c = blockIdx.x * 32 + threadIdx.x, b = blockIdx.y;
    const int len = min(lens[b], S);
    const int hist = taps - 1;
    Tin* st = state + (long)slots[b] * hist * C;
    const Tin* xb = x + (long)b * x_sb;
    if (c < C) {
        float wr[kMaxTaps];
#pragma unroll
        for (int j = 0; j < kMaxTaps; ++j) wr[j] = j < taps ? w[(long)c * taps + j] : 0.f;
        const float bc = bias ? bias[c] : 0.f;
        for (int t = threadIdx.y; t < S; t += blockDim.y) {
            float acc = 0.f;
            if (t < len) {
                acc = bc;
#pragma unroll
                for (int j = 0; j < kMaxTaps; ++j) {
                    if (j < taps) {
                        const int s = t - hist + j;
                        float v = 0.f;
                        if (s >= 0) v = ldf(xb + (long)s * x_st + c);
                        else if (!fresh) v = ldf(st + (long)(hist + s) * C + c);
                        acc = fmaf(wr[j], v, acc);
                    }
                }
                if (residual) acc += ldf(xb + (long)t * x_st + c);
            }
            stf(out + ((long)b * S + t) * C + c, acc);
        }
    }
    __syncthreads();   // every read of the old history is done before it is replaced
    if (threadIdx.y == 0 && c < C && hist > 0) {
        float nh[kMaxTaps];
#pragma unroll
        for (int i = 0; i < kMaxTaps - 1; ++i) {
            nh[i] = 0.f;
            if (i < hist) {
                const int s = len - hist + i;
                if (s >= 0) nh[i] = ldf(xb + (long)s * x_st + c);
                else if (!fresh) nh[i] = ldf(st + (long)(hist + s) * C + c);
            }
        }
#pragma unroll
        for (int i = 0; i < kMaxTaps - 1; ++i)
            if (i < hist) stf(st + (long)i * C + c, nh[i]);
    }
}

template <typename Tin, typename Tout>
static void launch(const void* x, long x_sb, long x_st, const float* w, const float* bias, void* state, const int* slots,
                   const int* lens, int B, int S, int C, int taps, int fresh, int residual, void* out, cudaStream_t s) {
    int ty = S >= 16 ? 16 : (S >= 4 ? 4 : 1);
    dim3 grid((C + 31) / 32, B), block(32, ty);
    short_conv_kernel<Tin, Tout><<<grid, block, 0, s>>>((const Tin*)x, x_sb, x_st, w, bias, (Tin*)state, slots, lens, S, C, taps,
                                                       fresh, residual, (Tout*)out);
}

void short_conv(const void* x, int in_bf16, long x_sb, long x_st, const float* w, const float* bias, void* state, const int* slots,
                const int* lens, int B, int S, int C, int taps, int fresh, int residual, void* out, int out_bf16, cudaStream_t s) {
    if (in_bf16 && out_bf16) launch<bf16, bf16>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, out, s);
    else if (!in_bf16 && out_bf16) launch<float, bf16>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, out, s);
    else if (!in_bf16 && !out_bf16) launch<float, float>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, out, s);
    else launch<bf16, float>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, out, s);
}

}  // namespace seqmix
