// Gated linear recurrences carried from token to token, states in float.
//   gla_scan  : per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, with a decay per KEY channel
//               alpha = sigmoid(z + bias)^(1/tau) = exp(log_sigmoid(z + bias) / tau), formed here in float from the projected z.
//               A block owns one (sequence, head, slice of value columns); a thread owns DPT rows of one state column in registers;
//               the step's alpha / k / q / v are staged through shared memory (double buffered: one barrier per token).
//   rglru_scan: per channel  a = exp(-8 r softplus(lam)),  h_t = a h_(t-1) + sqrt(1 - a^2) i u_t,  out = h_t * gelu_tanh(y)
//               with r, i = sigmoid(gate pre-activations + bias); sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)).
// Tokens at or past lens[b] are padding: they write zeros and do not touch the state.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kStage = 8;   // staged loads per thread and token

template <typename T, int DPT>
__global__ void gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long sb, long st,
                                const T* __restrict__ z, long z_sb, long z_st, const float* __restrict__ zbias, float inv_tau,
                                float qscale, float* state, const int* __restrict__ slots, const int* __restrict__ lens, int fresh,
                                int S, int H, int D, int V, int R, int Vb, float* __restrict__ out) {
    extern __shared__ float sm[];
    const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * Vb;
    const int tid = threadIdx.x, nthr = blockDim.x, r = tid % R, j = j0 + tid / R;
    const int len = min(lens[b], S), per = 3 * D + Vb;
    const bool live = tid / R < Vb && j < V;
    float s[DPT];
    float* sp = state + (((long)slots[b] * H + h) * D) * V;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = r + i * R;
        s[i] = (!fresh && live && d < D) ? sp[(long)d * V + j] : 0.f;
    }
    const long hq = (long)h * D, hv = (long)h * V + j0;
    auto fetch = [&](int t, int e) -> float {
        const long tok = (long)b * sb + (long)t * st;
        if (e < D) {
            float zz = ldf(z + (long)b * z_sb + (long)t * z_st + hq + e) + zbias[hq + e];
            return 1.f + expm1f(log_sigmoidf_(zz) * inv_tau);   // rounds once from an accurate value: no bias as alpha -> 1
        }
        if (e < 2 * D) return ldf(k + tok + hq + e - D);
        if (e < 3 * D) return ldf(q + tok + hq + e - 2 * D) * qscale;
        return (j0 + e - 3 * D < V) ? ldf(v + tok + hv + e - 3 * D) : 0.f;
    };
    if (len > 0)
        for (int e = tid; e < per; e += nthr) sm[e] = fetch(0, e);
    for (int t = 0; t < len; ++t) {
        float* cur = sm + (t & 1) * per;
        float* nxt = sm + ((t + 1) & 1) * per;
        __syncthreads();
        float stage[kStage];
        if (t + 1 < len) {
#pragma unroll
            for (int x = 0; x < kStage; ++x) {
                const int e = tid + x * nthr;
                stage[x] = e < per ? fetch(t + 1, e) : 0.f;
            }
        }
        const float vj = live ? cur[3 * D + tid / R] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r + i * R;
            if (d < D) {
                s[i] = fmaf(cur[d], s[i], cur[D + d] * vj);
                acc = fmaf(s[i], cur[2 * D + d], acc);
            }
        }
        for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (r == 0 && live) out[(((long)b * S + t) * H + h) * V + j] = acc;
        if (t + 1 < len) {
#pragma unroll
            for (int x = 0; x < kStage; ++x) {
                const int e = tid + x * nthr;
                if (e < per) nxt[e] = stage[x];
            }
        }
    }
    if (r == 0 && live)
        for (int t = len; t < S; ++t) out[(((long)b * S + t) * H + h) * V + j] = 0.f;
    if (live) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r + i * R;
            if (d < D) sp[(long)d * V + j] = s[i];
        }
    }
}

static int pow2ceil(int x) { int p = 1; while (p < x) p <<= 1; return p; }

template <typename T>
static bool gla_launch(const void* q, const void* k, const void* v, long sb, long st, const void* z, long z_sb, long z_st,
                       const float* zbias, float inv_tau, float qscale, float* state, const int* slots, const int* lens, int fresh,
                       int B, int S, int H, int D, int V, float* out, cudaStream_t s) {
    const int dpts[3] = {8, 16, 32};
    for (int a = 0; a < 3; ++a) {
        const int DPT = dpts[a], R = pow2ceil((D + DPT - 1) / DPT);
        if (R > 32) continue;
        int Vb = 256 / R; if (Vb < 1) Vb = 1; if (Vb > V) Vb = V;
        int threads = R * Vb;
        threads = ((threads + 31) / 32) * 32;
        if (3 * D + Vb > kStage * threads) continue;
        dim3 grid(H, B, (V + Vb - 1) / Vb);
        const size_t smem = 2 * (size_t)(3 * D + Vb) * sizeof(float);
#define SEQMIX_GLA(P)                                                                                                             \
    gla_scan_kernel<T, P><<<grid, threads, smem, s>>>((const T*)q, (const T*)k, (const T*)v, sb, st, (const T*)z, z_sb, z_st, zbias,  \
                                                      inv_tau, qscale, state, slots, lens, fresh, S, H, D, V, R, Vb, out)
        if (DPT == 8) SEQMIX_GLA(8); else if (DPT == 16) SEQMIX_GLA(16); else SEQMIX_GLA(32);
#undef SEQMIX_GLA
        return true;
    }
    return false;
}

bool gla_scan(const void* q, const void* k, const void* v, int bf, long sb, long st, const void* z, long z_sb, long z_st,
              const float* zbias, float inv_tau, float qscale, float* state, const int* slots, const int* lens, int fresh, int B, int S,
              int H, int D, int V, float* out, cudaStream_t s) {
    return bf ? gla_launch<bf16>(q, k, v, sb, st, z, z_sb, z_st, zbias, inv_tau, qscale, state, slots, lens, fresh, B, S, H, D, V, out, s)
              : gla_launch<float>(q, k, v, sb, st, z, z_sb, z_st, zbias, inv_tau, qscale, state, slots, lens, fresh, B, S, H, D, V, out, s);
}

template <typename T>
__global__ void rglru_scan_kernel(const T* __restrict__ u, const float* __restrict__ gr, const float* __restrict__ gi, int wb,
                                  const float* __restrict__ rbias, const float* __restrict__ ibias, const float* __restrict__ lam_sp,
                                  const T* __restrict__ y, long y_sb, long y_st, float* state, const int* __restrict__ slots,
                                  const int* __restrict__ lens, int fresh, int B, int S, int W, T* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= W) return;
    const int len = min(lens[b], S);
    const long N = (long)B * S;
    const long gbase = ((long)(c / wb) * N + (long)b * S) * wb + c % wb;       // gates are laid out [block, token, channel in block]
    const float rb = rbias[c], ib = ibias[c], sp = lam_sp[c];
    float* hs = state + (long)slots[b] * W + c;
    float h = fresh ? 0.f : *hs;
#pragma unroll 4
    for (int t = 0; t < len; ++t) {
        const float r = sigmoidf_(gr[gbase + (long)t * wb] + rb), g = sigmoidf_(gi[gbase + (long)t * wb] + ib);
        const float uu = ldf(u + ((long)b * S + t) * W + c), yy = ldf(y + (long)b * y_sb + (long)t * y_st + c);
        const float la = -8.f * r * sp, a = 1.f + expm1f(la), mult = sqrtf(-expm1f(2.f * la));
        h = fmaf(a, h, mult * g * uu);
        const float gl = 0.5f * yy * (1.f + tanhf(0.7978845608028654f * (yy + 0.044715f * yy * yy * yy)));
        stf(out + ((long)b * S + t) * W + c, h * gl);
    }
    for (int t = len; t < S; ++t) stf(out + ((long)b * S + t) * W + c, 0.f);
    *hs = h;
}

void rglru_scan(const void* u, int bf, const float* gr, const float* gi, int wb, const float* rbias, const float* ibias,
                const float* lam_sp, const void* y, long y_sb, long y_st, float* state, const int* slots, const int* lens, int fresh,
                int B, int S, int W, void* out, cudaStream_t s) {
    dim3 block(128), grid((W + 127) / 128, B);
    if (bf) rglru_scan_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)u, gr, gi, wb, rbias, ibias, lam_sp, (const bf16*)y, y_sb, y_st,
                                                          state, slots, lens, fresh, B, S, W, (bf16*)out);
    else rglru_scan_kernel<float><<<grid, block, 0, s>>>((const float*)u, gr, gi, wb, rbias, ibias, lam_sp, (const float*)y, y_sb, y_st,
                                                         state, slots, lens, fresh, B, S, W, (float*)out);
}

}  // namespace seqmix
