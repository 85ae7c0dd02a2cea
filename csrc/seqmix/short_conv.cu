// Causal depthwise convolution over time with a carried history ("short convolution"): used as the residual input convolution of
// every sublayer (out = h + conv(h)) and as the plain convolution of the recurrent block (out = conv(h) + bias).
//   out[b,t,c] = sum_j w[c,j] * in(b, t - taps + 1 + j, c),   in(b,s,c) = x[b,s,c] for s >= 0, else the slot's history (zeros when
// the sequence starts in this call).  After the call the slot's history holds the last taps-1 inputs of the sequence (positions
// beyond lens[b] are padding: they produce zeros and never enter the history).
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kMaxTaps = 16;

// silu of the convolution's result: the exact-rounded form for float outputs, fast exponential and division when the result is
// rounded to bfloat16 anyway
template <typename Tout> __device__ __forceinline__ float silu_out(float z);
template <> __device__ __forceinline__ float silu_out<float>(float z) { return z * sigmoidf_(z); }
template <> __device__ __forceinline__ float silu_out<bf16>(float z) { return __fdividef(z, 1.f + __expf(-z)); }

template <typename Tin, typename Tout>
__global__ void short_conv_kernel(const Tin* __restrict__ x, long x_sb, long x_st, const float* __restrict__ w,
                                  const float* __restrict__ bias, Tin* state, const int* __restrict__ slots,
                                  const int* __restrict__ lens, int S, int C, int taps, int fresh, int residual, int act,
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
                if (act) acc = silu_out<Tout>(acc);
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

// Vector form (taps <= 8, channels and strides multiples of 4, 16-byte aligned): a thread owns 4 channels and a run of 8 consecutive
// tokens, keeps the previous taps-1 inputs in registers and reads every input once.  A block covers 128 channels x 64 tokens; only
// the block of the first 64 tokens can touch the carried history, and it replaces it after its own reads.
constexpr int kVecTaps = 8, kRun = 8;

// VT: taps the registers are laid out for (4 or 8; the real count is an argument)
template <typename Tin, typename Tout, int VT>
__global__ void short_conv_vec_kernel(const Tin* __restrict__ x, long x_sb, long x_st, const float* __restrict__ w,
                                      const float* __restrict__ bias, Tin* state, const int* __restrict__ slots,
                                      const int* __restrict__ lens, int S, int C, int taps, int fresh, int residual, int act,
                                      Tout* __restrict__ out) {
    const int c = (blockIdx.x * 32 + threadIdx.x) * 4, b = blockIdx.z, tbase = blockIdx.y * (kRun * 8) + threadIdx.y * kRun;
    const int len = min(lens[b], S), hist = taps - 1;
    Tin* st = state + (long)slots[b] * hist * C;
    const Tin* xb = x + (long)b * x_sb;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    auto in4 = [&](int s) -> float4 {
        if (s >= 0) return ld4(xb + (long)s * x_st + c);
        if (!fresh) return ld4(st + (long)(hist + s) * C + c);
        return zero;
    };
    if (c < C) {
        float4 wr[VT], prev[VT - 1];          // right-aligned: wr[VT-1] weighs the current token
#pragma unroll
        for (int k = 0; k < VT; ++k) {
            const int j = k - (VT - taps);
            wr[k] = j >= 0 ? make_float4(w[(long)c * taps + j], w[(long)(c + 1) * taps + j], w[(long)(c + 2) * taps + j], w[(long)(c + 3) * taps + j]) : zero;
        }
        const float4 bc = bias ? ld4(bias + c) : zero;
#pragma unroll
        for (int k = 0; k < VT - 1; ++k) {
            const int s = tbase - (VT - 1) + k;
            prev[k] = (k >= VT - 1 - hist && tbase < len) ? in4(s) : zero;
        }
        float4 run[kRun];                                 // the run's own inputs, all loads in flight together
#pragma unroll
        for (int tt = 0; tt < kRun; ++tt) run[tt] = tbase + tt < len ? ld4(xb + (long)(tbase + tt) * x_st + c) : zero;
#pragma unroll
        for (int tt = 0; tt < kRun; ++tt) {
            const int t = tbase + tt;
            if (t < S) {
                float4 acc = zero;
                const float4 cur = run[tt];
                if (t < len) {
                    acc = bc;
#pragma unroll
                    for (int k = 0; k < VT - 1; ++k) {
                        acc.x = fmaf(wr[k].x, prev[k].x, acc.x); acc.y = fmaf(wr[k].y, prev[k].y, acc.y);
                        acc.z = fmaf(wr[k].z, prev[k].z, acc.z); acc.w = fmaf(wr[k].w, prev[k].w, acc.w);
                    }
                    const float4 wl = wr[VT - 1];
                    acc.x = fmaf(wl.x, cur.x, acc.x); acc.y = fmaf(wl.y, cur.y, acc.y);
                    acc.z = fmaf(wl.z, cur.z, acc.z); acc.w = fmaf(wl.w, cur.w, acc.w);
                    if (residual) { acc.x += cur.x; acc.y += cur.y; acc.z += cur.z; acc.w += cur.w; }
                    if (act) { acc.x = silu_out<Tout>(acc.x); acc.y = silu_out<Tout>(acc.y); acc.z = silu_out<Tout>(acc.z); acc.w = silu_out<Tout>(acc.w); }
                }
                st4(out + ((long)b * S + t) * C + c, acc);
#pragma unroll
                for (int k = 0; k < VT - 2; ++k) prev[k] = prev[k + 1];
                prev[VT - 2] = cur;
            }
        }
    }
    if (blockIdx.y != 0) return;
    __syncthreads();   // every read of the old history is done before it is replaced
    if (threadIdx.y == 0 && c < C && hist > 0) {
        float4 nh[VT - 1];
#pragma unroll
        for (int i = 0; i < VT - 1; ++i) nh[i] = i < hist ? in4(len - hist + i) : zero;
#pragma unroll
        for (int i = 0; i < VT - 1; ++i)
            if (i < hist) st4(st + (long)i * C + c, nh[i]);
    }
}

template <typename Tin, typename Tout>
static void launch(const void* x, long x_sb, long x_st, const float* w, const float* bias, void* state, const int* slots,
                   const int* lens, int B, int S, int C, int taps, int fresh, int residual, int act, void* out, cudaStream_t s) {
    const bool vec = taps <= kVecTaps && C % 4 == 0 && x_sb % 4 == 0 && x_st % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (uintptr_t)state % 16 == 0 && (!bias || (uintptr_t)bias % 16 == 0);
    if (vec) {
        dim3 grid((C / 4 + 31) / 32, (S + kRun * 8 - 1) / (kRun * 8), B), block(32, 8);
        if (taps <= 4)
            short_conv_vec_kernel<Tin, Tout, 4><<<grid, block, 0, s>>>((const Tin*)x, x_sb, x_st, w, bias, (Tin*)state, slots, lens, S, C, taps,
                                                                      fresh, residual, act, (Tout*)out);
        else
            short_conv_vec_kernel<Tin, Tout, 8><<<grid, block, 0, s>>>((const Tin*)x, x_sb, x_st, w, bias, (Tin*)state, slots, lens, S, C, taps,
                                                                      fresh, residual, act, (Tout*)out);
        return;
    }
    int ty = S >= 16 ? 16 : (S >= 4 ? 4 : 1);
    dim3 grid((C + 31) / 32, B), block(32, ty);
    short_conv_kernel<Tin, Tout><<<grid, block, 0, s>>>((const Tin*)x, x_sb, x_st, w, bias, (Tin*)state, slots, lens, S, C, taps,
                                                       fresh, residual, act, (Tout*)out);
}

void short_conv(const void* x, int in_bf16, long x_sb, long x_st, const float* w, const float* bias, void* state, const int* slots,
                const int* lens, int B, int S, int C, int taps, int fresh, int residual, int act, void* out, int out_bf16, cudaStream_t s) {
    if (in_bf16 && out_bf16) launch<bf16, bf16>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, act, out, s);
    else if (!in_bf16 && out_bf16) launch<float, bf16>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, act, out, s);
    else if (!in_bf16 && !out_bf16) launch<float, float>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, act, out, s);
    else launch<bf16, float>(x, x_sb, x_st, w, bias, state, slots, lens, B, S, C, taps, fresh, residual, act, out, s);
}

}  // namespace seqmix
