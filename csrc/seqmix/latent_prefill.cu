// Latent sliding-window attention over a prompt, expanded form, as one fused kernel (bfloat16 operands): scores, window mask,
// softmax and the weighted sum of values never leave the chip.  A block owns 64 consecutive queries of one (sequence, head); its four
// warps own 16 queries each.  Key / value tiles of 64 positions are staged in shared memory by asynchronous copies, one tile ahead
// of the arithmetic; a head's key row is its own unrotated part (from the expanded keys) followed by the rotated part that all heads
// share (from the prepared latent rows).  Scores come from
// tensor-core products (mma.sync m16n8k16, float accumulation), are scaled, masked and exponentiated in float with a running maximum
// and sum per query; the weights are rounded to bfloat16 only as operands of the value product, whose accumulator is float.
// Position i sees j with 0 <= i - j < window.  Queries at or past lens[b] give zeros.
// Sizes: key and value sizes are multiples of 16 up to 16 * DK16 / 16 * VD16 (template bounds; the real sizes are arguments).
#include "mma_tiles.cuh"
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kQT = 64, kKT = 64, kPad = 8;     // queries / keys per tile; row padding (elements) against bank conflicts

// q [B,S,H,DK]; kx [B,S,H,D] unrotated keys; rows [B,S,CR] whose last R numbers are the shared rotated key part; v [B,S,H,VD];
// out [B,S,H*VD].  DK = D + R.
template <int DK16, int VD16>
__global__ void __launch_bounds__(128)
latent_prompt_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kx, const bf16* __restrict__ rows, const bf16* __restrict__ v,
                          const int* __restrict__ lens, int S, int H, int D, int R, int CR, int VD, int window, float scale,
                          bf16* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DK = D + R, dk16 = DK / 16, vd16 = VD / 16, ldk = DK + kPad, ldv = VD + kPad;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [kQT][ldk] queries, then key stage 1 (same size)
    auto Kst = [&](int st) { return st ? Qs : Qs + kQT * ldk; };                               // [kKT][ldk] each
    auto Vst = [&](int st) { return Qs + (kQT + kKT) * ldk + (st ? kKT * ldv : 0); };          // [kKT][ldv] each
    const int q0 = blockIdx.x * kQT, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int len = min(lens[b], S);
    bf16* ob = out + ((long)b * S) * H * VD + (long)h * VD;
    if (q0 >= len) {                                       // nothing but padding: zeros
        for (int i = tid; i < min(kQT, S - q0) * (VD / 2); i += 128) {
            const int r = i / (VD / 2), c = (i % (VD / 2)) * 2;
            *reinterpret_cast<unsigned*>(ob + (long)(q0 + r) * H * VD + c) = 0u;
        }
        return;
    }
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    // queries of the tile (rows past the sequence: zeros)
    for (int i = tid; i < kQT * (DK / 8); i += 128) {
        const int r = i / (DK / 8), c = (i % (DK / 8)) * 8, t = q0 + r;
        *reinterpret_cast<uint4*>(Qs + r * ldk + c) = t < S ? *reinterpret_cast<const uint4*>(q + (((long)b * S + t) * H + h) * DK + c) : zero4;
    }
    __syncthreads();
    const int r0 = warp * 16, g = lane >> 2, tq = lane & 3;
    unsigned qa[DK16][4];
#pragma unroll
    for (int kk = 0; kk < DK16; ++kk)
        if (kk < dk16) ldsm4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], Qs + (r0 + (lane & 15)) * ldk + kk * 16 + (lane >> 4) * 8);
    float oacc[2 * VD16][4];
#pragma unroll
    for (int n = 0; n < 2 * VD16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int i0 = q0 + r0 + g, i1 = i0 + 8;               // this thread's two queries
    const float scale2 = scale * 1.4426950408889634f;
    const int jlo = max(0, q0 - window + 1), jhi = min(q0 + kQT - 1, len - 1);
    // key / value tiles arrive by asynchronous copies, one tile ahead of the arithmetic (two stages)
    auto fetch = [&](int kt, int st) {
        const int j0 = kt * kKT;
        bf16 *Kd = Kst(st), *Vd = Vst(st);
        // a warp per key row and pass, a lane per 16-byte piece (cheap index arithmetic: this runs once per tile and thread)
        for (int c = lane * 8; c < DK; c += 256) {
            const bool lo = c < D;
            const long off = lo ? (long)h * D + c : (long)(CR - R) + (c - D), stride = lo ? (long)H * D : (long)CR;
            const bf16* base = (lo ? kx : rows) + (long)b * S * stride + off;
#pragma unroll 4
            for (int r = warp; r < kKT; r += 4) {
                const int j = j0 + r;
                cp16(Kd + r * ldk + c, base + (long)min(j, len - 1) * stride, j < len);
            }
        }
        for (int c = lane * 8; c < VD; c += 256) {
            const bf16* base = v + ((long)b * S * H + h) * VD + c;
#pragma unroll 4
            for (int r = warp; r < kKT; r += 4) {
                const int j = j0 + r;
                cp16(Vd + r * ldv + c, base + (long)min(j, len - 1) * H * VD, j < len);
            }
        }
        cp_commit();
    };
    const int kt0 = jlo / kKT, kt1 = jhi / kKT;
    __syncthreads();                                       // every warp holds its queries: their room becomes key stage 1
    fetch(kt0, 0);
    for (int kt = kt0; kt <= kt1; ++kt) {
        const int j0 = kt * kKT, st = (kt - kt0) & 1;
        if (kt < kt1) { fetch(kt + 1, st ^ 1); cp_wait<1>(); } else cp_wait<0>();
        __syncthreads();                                   // tile kt has landed for everyone
        const bf16 *Ks = Kst(st), *Vs = Vst(st);
        float sacc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DK16; ++kk) {
            if (kk < dk16) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {           // two 8-key groups per ldmatrix
                    unsigned b0, b1, b2, b3;
                    ldsm4(b0, b1, b2, b3, Ks + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma16816(sacc[2 * np], qa[kk], b0, b1);
                    mma16816(sacc[2 * np + 1], qa[kk], b2, b3);
                }
            }
        }
        // scale, mask, running softmax (float, in base 2: scores carry scale * log2(e)); a thread holds 16 scores of query i0 and 16
        // of i1.  A tile that every query of the warp sees in full needs no mask.
        const int wlo = q0 + r0, whi = wlo + 15;
        const bool full = j0 + kKT - 1 <= wlo && j0 > whi - window && j0 + kKT - 1 < len;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                bool vis = true;
                if (!full) {
                    const int j = j0 + n * 8 + tq * 2 + (e & 1), i = (e < 2) ? i0 : i1;
                    vis = j <= i && j > i - window && j < len;
                }
                sacc[n][e] = vis ? sacc[n][e] * scale2 : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], sacc[n][e]);
            }
        float corr[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(mrow[r], mx[r]);
            base[r] = mn == -INFINITY ? 0.f : mn;          // nothing visible so far: every weight is exp(-inf) = 0
            corr[r] = exp2f(mrow[r] - base[r]);
            mrow[r] = mn;
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sacc[n][e] = exp2f(sacc[n][e] - base[e >> 1]);
                ls[e >> 1] += sacc[n][e];
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * corr[r] + ls[r];
#pragma unroll
        for (int n = 0; n < 2 * VD16; ++n) { oacc[n][0] *= corr[0]; oacc[n][1] *= corr[0]; oacc[n][2] *= corr[1]; oacc[n][3] *= corr[1]; }
        // weighted values: 4 steps of 16 keys
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {
            unsigned pa[4];
            pa[0] = pack2(sacc[2 * kp][0], sacc[2 * kp][1]);
            pa[1] = pack2(sacc[2 * kp][2], sacc[2 * kp][3]);
            pa[2] = pack2(sacc[2 * kp + 1][0], sacc[2 * kp + 1][1]);
            pa[3] = pack2(sacc[2 * kp + 1][2], sacc[2 * kp + 1][3]);
#pragma unroll
            for (int nv = 0; nv < VD16; ++nv) {
                if (nv < vd16) {
                    unsigned b0, b1, b2, b3;
                    ldsm4t(b0, b1, b2, b3, Vs + (kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + nv * 16 + (lane >> 4) * 8);
                    mma16816(oacc[2 * nv], pa, b0, b1);
                    mma16816(oacc[2 * nv + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();                                   // the stage may be refilled
    }
    // the quad's partial sums of weights meet; normalise and write
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
    const float inv0 = (i0 < len && lrow[0] > 0.f) ? 1.f / lrow[0] : 0.f, inv1 = (i1 < len && lrow[1] > 0.f) ? 1.f / lrow[1] : 0.f;
#pragma unroll
    for (int n = 0; n < 2 * VD16; ++n) {
        if (n < 2 * vd16) {
            const int c = n * 8 + tq * 2;
            if (i0 < S) *reinterpret_cast<unsigned*>(ob + (long)i0 * H * VD + c) = pack2(oacc[n][0] * inv0, oacc[n][1] * inv0);
            if (i1 < S) *reinterpret_cast<unsigned*>(ob + (long)i1 * H * VD + c) = pack2(oacc[n][2] * inv1, oacc[n][3] * inv1);
        }
    }
}

bool latent_prompt_attention_fits(int D, int R, int CR, int VD) {
    const int DK = D + R;
    return DK % 16 == 0 && VD % 16 == 0 && D % 8 == 0 && R % 8 == 0 && CR % 8 == 0 && DK <= 256 && VD <= 256;
}

bool latent_prompt_attention(const void* q, const void* kx, const void* rows, const void* v, const int* lens, int B, int S, int H, int D,
                             int R, int CR, int VD, int window, float scale, void* out, cudaStream_t s) {
    if (!latent_prompt_attention_fits(D, R, CR, VD)) return false;
    const int DK = D + R;
    const size_t smem = (size_t)((kQT + kKT) * (DK + kPad) + 2 * kKT * (VD + kPad)) * sizeof(bf16);
    dim3 grid((S + kQT - 1) / kQT, H, B);
#define SEQMIX_LPA(A, Bv)                                                                                                           \
    do {                                                                                                                            \
        cudaFuncSetAttribute(latent_prompt_attn_kernel<A, Bv>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);            \
        latent_prompt_attn_kernel<A, Bv><<<grid, 128, smem, s>>>((const bf16*)q, (const bf16*)kx, (const bf16*)rows, (const bf16*)v, lens, \
                                                                S, H, D, R, CR, VD, window, scale, (bf16*)out);                     \
    } while (0)
    if (DK <= 64 && VD <= 64) SEQMIX_LPA(4, 4);
    else if (DK <= 128 && VD <= 128) SEQMIX_LPA(8, 8);
    else if (DK <= 192 && VD <= 128) SEQMIX_LPA(12, 8);
    else SEQMIX_LPA(16, 16);
#undef SEQMIX_LPA
    return true;
}

}  // namespace seqmix
