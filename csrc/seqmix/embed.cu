// Token embedding with a constant scale and interleaved sinusoids of the position added, written as the float residual stream:
//   out[b,t,c] = table[token[b,t], c] * scale + (c even ? sin : cos)((pos0[b] + t) * inv_freq[c / 2])       (angles in float)
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

template <typename T>
__global__ void embed_sinusoid_kernel(const long* __restrict__ tokens, const T* __restrict__ table, float scale,
                                      const float* __restrict__ inv_freq, const int* __restrict__ pos0, int S, int W, int vocab,
                                      float* __restrict__ out) {
    const long row = blockIdx.x;
    const int b = (int)(row / S), t = (int)(row - (long)b * S);
    const long tok = min(max(tokens[row], 0L), (long)vocab - 1);
    const float p = (float)(pos0[b] + t);
    const T* e = table + tok * W;
    float* o = out + row * W;
    for (int i = threadIdx.x; i < (W + 1) / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(p * inv_freq[i], &sn, &cs);
        o[2 * i] = fmaf(ldf(e + 2 * i), scale, sn);
        if (2 * i + 1 < W) o[2 * i + 1] = fmaf(ldf(e + 2 * i + 1), scale, cs);
    }
}

void embed_sinusoid(const long* tokens, const void* table, int bf, float scale, const float* inv_freq, const int* pos0, int B, int S, int W,
                    int vocab, float* out, cudaStream_t s) {
    if (B * S == 0) return;
    const int threads = W >= 512 ? 256 : 128;
    if (bf) embed_sinusoid_kernel<bf16><<<B * S, threads, 0, s>>>(tokens, (const bf16*)table, scale, inv_freq, pos0, S, W, vocab, out);
    else embed_sinusoid_kernel<float><<<B * S, threads, 0, s>>>(tokens, (const float*)table, scale, inv_freq, pos0, S, W, vocab, out);
}

}  // namespace seqmix
