// Latent sliding-window attention for single new tokens (decoding), absorbed form, split over the ring cache.
// One block = kChunk consecutive ring rows of one sequence x one tile of kHeads heads.  The block stages its ring rows in shared
// memory once (as floats) and uses them twice: as keys (scores of every head of the tile against every row; all heads share the
// rows) and as values (the weighted sum of the latents).  Each block leaves a partial softmax (running maximum, sum of weights,
// unnormalised weighted sum) per head; a second kernel merges the partials of a sequence's chunks and writes the result in the
// activation dtype.  Scores, weights and sums are float throughout.
// Ring row kk of a sequence at position p holds position j = p - ((p - kk) mod ring); it is visible when j >= 0 and p - j < window.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

static const int kChunk = 32;    // ring rows per block (one lane per row in the softmax step)
static const int kHeads = 8;     // heads per block
static const int kThreads = 512;
static const int kRowRegs = 20;  // row coordinates per lane: C + R <= 32 * kRowRegs
static const int kColsPerThread = 2;   // value columns per thread: C <= kColsPerThread * kThreads

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads, 2)
latent_ring_partial_kernel(const T* __restrict__ qa, long qa_sn, long qa_sh, const T* __restrict__ qr, long qr_sn, long qr_sh,
                           const T* __restrict__ keys, long key_sb, int ring, const int* __restrict__ key_index,
                           const int* __restrict__ pos0, const int* __restrict__ lens, int H, int C, int R, int window, float scale,
                           int nsplit, float* __restrict__ part_m, float* __restrict__ part_l, float* __restrict__ part_acc) {
    extern __shared__ float smem[];
    const int CR = C + R, CRp = (CR + 31) & ~31, nE = CRp / 32, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, b = blockIdx.y, h0 = blockIdx.z * kHeads, nh = min(kHeads, H - h0);
    float* sq = smem;                          // [kHeads][CRp]  (rows padded with zeros to whole 32s: no bounds in the inner loops)
    float* sk = sq + kHeads * CRp;             // [kChunk][CRp]
    float* sp = sk + kChunk * CRp;             // [kHeads][kChunk] scores
    float* sw = sp + kHeads * kChunk;          // [kChunk][kHeads] weights
    const int p = pos0[b], r0 = split * kChunk, nr = min(kChunk, ring - r0);
    const long pbase = ((long)b * nsplit + split) * H + h0;
    // which rows of this chunk are visible (the same for every head)
    auto visible = [&](int kk) -> bool {
        int m = (p - kk) % ring;
        if (m < 0) m += ring;
        return p - m >= 0 && m < window;
    };
    // one lane per ring row of the chunk: the mask of visible rows, the same in every warp
    const unsigned vismask = __ballot_sync(0xffffffffu, lens[b] > 0 && lane < nr && visible(r0 + lane));
    const bool any = vismask != 0u;
    if (!any) {                                // nothing to see here: an empty partial with weight zero
        if (tid < nh) { part_m[pbase + tid] = -INFINITY; part_l[pbase + tid] = 0.f; }
        for (int i = tid; i < nh * C; i += kThreads) part_acc[pbase * C + i] = 0.f;
        return;
    }
    const T* base = keys + (long)(key_index ? key_index[b] : b) * key_sb + (long)r0 * CR;
    if (nh < kHeads || CR != CRp) {            // heads past the tile's last and the rows' padding read as zeros
        for (int i = tid; i < (kHeads + kChunk) * CRp; i += kThreads) sq[i] = 0.f;
        __syncthreads();
    }
    if (VEC) {                                 // every extent and stride a multiple of four elements, aligned bases
        const int CR4 = CR / 4;
        constexpr int kBatch = 8;              // loads in flight per thread
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i0 = 0; i0 < nr * CR4; i0 += kBatch * kThreads) {
            float4 v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) { const int i = i0 + u * kThreads + tid; v[u] = i < nr * CR4 ? ld4(base + 4 * i) : zero; }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = i0 + u * kThreads + tid;
                if (i < nr * CR4) *reinterpret_cast<float4*>(sk + (i / CR4) * CRp + (i % CR4) * 4) = v[u];
            }
        }
        for (int i0 = 0; i0 < nh * CR4; i0 += kBatch * kThreads) {
            float4 v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = i0 + u * kThreads + tid, h = i / CR4, d = (i % CR4) * 4;
                v[u] = i >= nh * CR4 ? zero : (d < C ? ld4(qa + (long)b * qa_sn + (long)(h0 + h) * qa_sh + d)
                                                     : ld4(qr + (long)b * qr_sn + (long)(h0 + h) * qr_sh + d - C));
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = i0 + u * kThreads + tid;
                if (i < nh * CR4) *reinterpret_cast<float4*>(sq + (i / CR4) * CRp + (i % CR4) * 4) = v[u];
            }
        }
    } else {
        for (int i = tid; i < nr * CR; i += kThreads) sk[(i / CR) * CRp + i % CR] = ldf(base + i);
        for (int i = tid; i < nh * CR; i += kThreads) {
            const int h = i / CR, d = i % CR;
            sq[h * CRp + d] = d < C ? ldf(qa + (long)b * qa_sn + (long)(h0 + h) * qa_sh + d) : ldf(qr + (long)b * qr_sn + (long)(h0 + h) * qr_sh + d - C);
        }
    }
    __syncthreads();
    // scores: a warp per pair of ring rows (kept in registers), lanes over the coordinates, four heads at once
    for (int j0 = warp; j0 < nr; j0 += 2 * (kThreads / 32)) {
        const int j1 = j0 + kThreads / 32;
        const bool two = j1 < nr;
        float ka[kRowRegs], kb[kRowRegs];
#pragma unroll
        for (int e = 0; e < kRowRegs; ++e) {
            if (e < nE) {
                ka[e] = sk[j0 * CRp + e * 32 + lane];
                kb[e] = two ? sk[j1 * CRp + e * 32 + lane] : 0.f;
            }
        }
        for (int h = 0; h < nh; h += 4) {
            float pa[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < kRowRegs; ++e) {
                if (e < nE) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float qv = sq[(h + g) * CRp + e * 32 + lane];
                        pa[g] = fmaf(qv, ka[e], pa[g]);
                        pb[g] = fmaf(qv, kb[e], pb[g]);
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    pa[g] += __shfl_xor_sync(0xffffffffu, pa[g], o);
                    pb[g] += __shfl_xor_sync(0xffffffffu, pb[g], o);
                }
            if (lane < 4 && h + lane < nh) {
                sp[(h + lane) * kChunk + j0] = (lane == 0 ? pa[0] : lane == 1 ? pa[1] : lane == 2 ? pa[2] : pa[3]) * scale;
                if (two) sp[(h + lane) * kChunk + j1] = (lane == 0 ? pb[0] : lane == 1 ? pb[1] : lane == 2 ? pb[2] : pb[3]) * scale;
            }
        }
    }
    __syncthreads();
    // partial softmax: a warp per head, a lane per ring row (heads past the tile's last keep weight zero)
    for (int i = tid; i < kChunk * kHeads; i += kThreads) sw[i] = 0.f;
    __syncthreads();
    for (int h = warp; h < nh; h += kThreads / 32) {
        const bool vis = (vismask >> lane) & 1u;
        const float s = vis ? sp[h * kChunk + lane] : -INFINITY;
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float w = vis ? expf(s - mx) : 0.f;
        const float l = warp_sum(w);
        sw[lane * kHeads + h] = w;
        if (lane == 0) { part_m[pbase + h] = mx; part_l[pbase + h] = l; }
    }
    __syncthreads();
    // weighted sum of the latents: a thread per value column, all heads of the tile in registers
    float acc[kColsPerThread][kHeads];
#pragma unroll
    for (int e = 0; e < kColsPerThread; ++e)
#pragma unroll
        for (int h = 0; h < kHeads; ++h) acc[e][h] = 0.f;
    for (int j = 0; j < nr; ++j) {
        float kv[kColsPerThread];
#pragma unroll
        for (int e = 0; e < kColsPerThread; ++e) {
            const int c = tid + e * kThreads;
            kv[e] = c < C ? sk[j * CRp + c] : 0.f;
        }
        float w[kHeads];                          // the same addresses for the whole warp
#pragma unroll
        for (int h4 = 0; h4 < kHeads / 4; ++h4) {
            const float4 t = *reinterpret_cast<const float4*>(sw + j * kHeads + 4 * h4);
            w[4 * h4] = t.x; w[4 * h4 + 1] = t.y; w[4 * h4 + 2] = t.z; w[4 * h4 + 3] = t.w;
        }
#pragma unroll
        for (int h = 0; h < kHeads; ++h)
#pragma unroll
            for (int e = 0; e < kColsPerThread; ++e) acc[e][h] = fmaf(w[h], kv[e], acc[e][h]);
    }
#pragma unroll
    for (int e = 0; e < kColsPerThread; ++e) {
        const int c = tid + e * kThreads;
        if (c < C)
#pragma unroll
            for (int h = 0; h < kHeads; ++h)
                if (h < nh) part_acc[(pbase + h) * C + c] = acc[e][h];
    }
}

// grid (H, B): merges the chunk partials of one (sequence, head) and writes out[h, b, :].  The chunks' weights exp(m_s - M) / L are
// formed once (a lane per chunk) and kept in shared memory; every thread then sums its columns over the chunks, loads unrolled.
template <typename T>
__global__ void latent_ring_merge_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                         const float* __restrict__ part_acc, int nsplit, int H, int C, T* __restrict__ out, long out_sn,
                                         long out_sh) {
    extern __shared__ float sw[];              // [nsplit]
    __shared__ float red[2];
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const long i0 = (long)b * nsplit * H + h;  // partial of chunk s: i0 + s * H
    if (tid < 32) {
        float M = -INFINITY;
        for (int s = lane; s < nsplit; s += 32) M = fmaxf(M, part_m[i0 + (long)s * H]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
        for (int s = lane; s < nsplit; s += 32) {
            const float l = part_l[i0 + (long)s * H];
            const float w = l > 0.f ? expf(part_m[i0 + (long)s * H] - M) : 0.f;
            sw[s] = w;
            L = fmaf(l, w, L);
        }
        L = warp_sum(L);
        if (lane == 0) { red[0] = M; red[1] = L; }
    }
    __syncthreads();
    T* o = out + (long)b * out_sn + (long)h * out_sh;
    if (red[0] == -INFINITY) {                 // a padded row: nothing visible anywhere
        for (int c = tid; c < C; c += blockDim.x) stf(o + c, 0.f);
        return;
    }
    const float inv = 1.f / red[1];
    for (int c = tid; c < C; c += blockDim.x) {
        const float* pa = part_acc + i0 * C + c;
        float a = 0.f;
#pragma unroll 8
        for (int s = 0; s < nsplit; ++s) a = fmaf(pa[(long)s * H * C], sw[s], a);
        stf(o + c, a * inv);
    }
}

int latent_ring_decode_splits(int ring) { return (ring + kChunk - 1) / kChunk; }

bool latent_ring_decode_fits(int C, int R) {
    return C <= kColsPerThread * kThreads && C + R <= 32 * kRowRegs && (size_t)((kHeads + kChunk) * ((C + R + 31) & ~31) + 2 * kHeads * kChunk) * sizeof(float) <= 200 * 1024;
}

template <typename T>
static void ring_decode_launch(const void* qa, long qa_sn, long qa_sh, const void* qr, long qr_sn, long qr_sh, const void* keys, long key_sb,
                               int ring, const int* key_index, const int* pos0, const int* lens, int B, int H, int C, int R, int window,
                               float scale, float* part_m, float* part_l, float* part_acc, void* out, long out_sn, long out_sh,
                               cudaStream_t s) {
    const int nsplit = latent_ring_decode_splits(ring);
    const size_t smem = (size_t)((kHeads + kChunk) * ((C + R + 31) & ~31) + 2 * kHeads * kChunk) * sizeof(float);
    dim3 grid(nsplit, B, (H + kHeads - 1) / kHeads);
    const size_t a4 = 4 * sizeof(T);
    const bool vec = C % 4 == 0 && R % 4 == 0 && qa_sn % 4 == 0 && qa_sh % 4 == 0 && qr_sn % 4 == 0 && qr_sh % 4 == 0 && key_sb % 4 == 0 &&
                     (uintptr_t)qa % a4 == 0 && (uintptr_t)qr % a4 == 0 && (uintptr_t)keys % a4 == 0;
#define SEQMIX_RING(V)                                                                                                              \
    do {                                                                                                                            \
        cudaFuncSetAttribute(latent_ring_partial_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);            \
        latent_ring_partial_kernel<T, V><<<grid, kThreads, smem, s>>>((const T*)qa, qa_sn, qa_sh, (const T*)qr, qr_sn, qr_sh,        \
                                                                      (const T*)keys, key_sb, ring, key_index, pos0, lens, H, C, R,  \
                                                                      window, scale, nsplit, part_m, part_l, part_acc);             \
    } while (0)
    if (vec) SEQMIX_RING(true); else SEQMIX_RING(false);
#undef SEQMIX_RING
    const int mt = C >= 256 ? 256 : (C >= 128 ? 128 : 64);
    latent_ring_merge_kernel<T><<<dim3(H, B), mt, nsplit * sizeof(float), s>>>(part_m, part_l, part_acc, nsplit, H, C, (T*)out, out_sn, out_sh);
}

void latent_ring_decode(const void* qa, int bf, long qa_sn, long qa_sh, const void* qr, long qr_sn, long qr_sh, const void* keys,
                        long key_sb, int ring, const int* key_index, const int* pos0, const int* lens, int B, int H, int C, int R,
                        int window, float scale, float* part_m, float* part_l, float* part_acc, void* out, long out_sn, long out_sh,
                        cudaStream_t s) {
    if (bf) ring_decode_launch<bf16>(qa, qa_sn, qa_sh, qr, qr_sn, qr_sh, keys, key_sb, ring, key_index, pos0, lens, B, H, C, R, window, scale,
                                     part_m, part_l, part_acc, out, out_sn, out_sh, s);
    else ring_decode_launch<float>(qa, qa_sn, qa_sh, qr, qr_sn, qr_sh, keys, key_sb, ring, key_index, pos0, lens, B, H, C, R, window, scale,
                                   part_m, part_l, part_acc, out, out_sn, out_sh, s);
}

}  // namespace seqmix
