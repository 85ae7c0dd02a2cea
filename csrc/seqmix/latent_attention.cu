// Latent (compressed-KV) attention with a sliding window, in the "absorbed" form: per token only the normalised latent c (C numbers)
// and one rotated key part shared by all heads (R numbers) are kept.  A query head carries qa = W_uk^T q_unrotated (C numbers) and
// its rotated part (R numbers); score = (qa . c + q_rot . k_rot) * scale; the output is the softmax-weighted sum of the latents
// themselves (the value up-projection follows as a matrix product).  The same row of the key store therefore serves as key AND
// value, and is read once per (query, key) pair.
//   latent_kv_store : RMS-norm of the latent, rotation of the shared key part at the token's position, append to the ring cache
//   rope_q          : rotation of each head's rotated query part, in place
//   latent_window_attention : one warp per (token, head), lanes over the C+R coordinates, online softmax in float
// Position i sees j with 0 <= i - j < window.  The key store is addressed as row (j mod ring) of a sequence's block: a ring of
// `window` rows for decoding, or the rows of the running prompt (ring = padded prompt length) for a prompt that starts at 0.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

template <typename T>
__global__ void latent_kv_store_kernel(const T* __restrict__ kv, long kv_sb, long kv_st, int B, int S, int C, int R, int dims,
                                       const float* __restrict__ nw, float eps, const float* __restrict__ inv_freq,
                                       const int* __restrict__ pos0, const int* __restrict__ lens, const int* __restrict__ slots,
                                       T* __restrict__ cache, int ring, T* __restrict__ rows) {
    const int n = blockIdx.x * blockDim.y + threadIdx.y, lane = threadIdx.x;
    if (n >= B * S) return;
    const int b = n / S, t = n % S, len = min(lens[b], S);
    if (t >= len) return;
    const int p = pos0[b] + t, CR = C + R, half = dims / 2;
    const T* x = kv + (long)b * kv_sb + (long)t * kv_st;
    T* dst_row = rows ? rows + (long)n * CR : nullptr;
    T* dst_cache = (cache && t >= len - ring) ? cache + ((long)slots[b] * ring + (p % ring)) * CR : nullptr;
    float ss = 0.f;
    for (int c = lane; c < C; c += 32) { float v = ldf(x + c); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)C + eps);
    for (int c = lane; c < C; c += 32) {
        float v = ldf(x + c) * inv * nw[c];
        if (dst_row) stf(dst_row + c, v);
        if (dst_cache) stf(dst_cache + c, v);
    }
    for (int i = lane; i < half; i += 32) {
        float u = ldf(x + C + i), v = ldf(x + C + i + half), sn, cs;
        sincosf((float)p * inv_freq[i], &sn, &cs);
        float a = u * cs - v * sn, bb = v * cs + u * sn;
        if (dst_row) { stf(dst_row + C + i, a); stf(dst_row + C + i + half, bb); }
        if (dst_cache) { stf(dst_cache + C + i, a); stf(dst_cache + C + i + half, bb); }
    }
    for (int i = dims + lane; i < R; i += 32) {      // coordinates past the rotated ones pass unchanged
        float v = ldf(x + C + i);
        if (dst_row) stf(dst_row + C + i, v);
        if (dst_cache) stf(dst_cache + C + i, v);
    }
}

template <typename T>
__global__ void rope_q_kernel(T* __restrict__ q, long q_sn, long q_sh, int N, int S, int H, int dims,
                              const float* __restrict__ inv_freq, const int* __restrict__ pos0) {
    const int half = dims / 2;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)N * H * half) return;
    const int i = idx % half, h = (idx / half) % H, n = idx / ((long)half * H);
    const int p = pos0[n / S] + n % S;
    T* x = q + (long)n * q_sn + (long)h * q_sh;
    float u = ldf(x + i), v = ldf(x + i + half), sn, cs;
    sincosf((float)p * inv_freq[i], &sn, &cs);
    stf(x + i, u * cs - v * sn);
    stf(x + i + half, v * cs + u * sn);
}

// Vector forms of the two kernels above (every extent, stride and offset a multiple of four elements, 16-byte aligned bases): a
// lane handles four consecutive coordinates per step and keeps the latent in registers between the statistic and the scaling.
constexpr int kStoreVec = 8;        // float4 per lane: latents up to 1024 numbers

template <typename T>
__global__ void latent_kv_store_vec_kernel(const T* __restrict__ kv, long kv_sb, long kv_st, int B, int S, int C, int R, int dims,
                                           const float* __restrict__ nw, float eps, const float* __restrict__ inv_freq,
                                           const int* __restrict__ pos0, const int* __restrict__ lens, const int* __restrict__ slots,
                                           T* __restrict__ cache, int ring, T* __restrict__ rows) {
    const int n = blockIdx.x * blockDim.y + threadIdx.y, lane = threadIdx.x;
    if (n >= B * S) return;
    const int b = n / S, t = n % S, len = min(lens[b], S);
    if (t >= len) return;
    const int p = pos0[b] + t, CR = C + R, half = dims / 2;
    const T* x = kv + (long)b * kv_sb + (long)t * kv_st;
    T* dst_row = rows ? rows + (long)n * CR : nullptr;
    T* dst_cache = (cache && t >= len - ring) ? cache + ((long)slots[b] * ring + (p % ring)) * CR : nullptr;
    float4 v[kStoreVec];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < kStoreVec; ++e) {
        const int c = (e * 32 + lane) * 4;
        v[e] = c < C ? ld4(x + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[e].x, v[e].x, fmaf(v[e].y, v[e].y, fmaf(v[e].z, v[e].z, fmaf(v[e].w, v[e].w, ss))));
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)C + eps);
#pragma unroll
    for (int e = 0; e < kStoreVec; ++e) {
        const int c = (e * 32 + lane) * 4;
        if (c < C) {
            const float4 g = ld4(nw + c);
            const float4 o = make_float4(v[e].x * inv * g.x, v[e].y * inv * g.y, v[e].z * inv * g.z, v[e].w * inv * g.w);
            if (dst_row) st4(dst_row + c, o);
            if (dst_cache) st4(dst_cache + c, o);
        }
    }
    for (int i = lane * 4; i < half; i += 128) {
        const float4 u = ld4(x + C + i), w = ld4(x + C + i + half), f = ld4(inv_freq + i);
        float4 sn, cs;
        sincosf((float)p * f.x, &sn.x, &cs.x); sincosf((float)p * f.y, &sn.y, &cs.y);
        sincosf((float)p * f.z, &sn.z, &cs.z); sincosf((float)p * f.w, &sn.w, &cs.w);
        const float4 a = make_float4(u.x * cs.x - w.x * sn.x, u.y * cs.y - w.y * sn.y, u.z * cs.z - w.z * sn.z, u.w * cs.w - w.w * sn.w);
        const float4 bb = make_float4(w.x * cs.x + u.x * sn.x, w.y * cs.y + u.y * sn.y, w.z * cs.z + u.z * sn.z, w.w * cs.w + u.w * sn.w);
        if (dst_row) { st4(dst_row + C + i, a); st4(dst_row + C + i + half, bb); }
        if (dst_cache) { st4(dst_cache + C + i, a); st4(dst_cache + C + i + half, bb); }
    }
    for (int i = dims + lane; i < R; i += 32) {      // coordinates past the rotated ones pass unchanged
        float u = ldf(x + C + i);
        if (dst_row) stf(dst_row + C + i, u);
        if (dst_cache) stf(dst_cache + C + i, u);
    }
}

template <typename T>
__global__ void rope_q_vec_kernel(T* __restrict__ q, long q_sn, long q_sh, int N, int S, int H, int dims,
                                  const float* __restrict__ inv_freq, const int* __restrict__ pos0) {
    const int quads = dims / 8;                      // groups of four pairs per head
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)N * H * quads) return;
    const int i = (int)(idx % quads) * 4, h = (idx / quads) % H, n = idx / ((long)quads * H), half = dims / 2;
    const int p = pos0[n / S] + n % S;
    T* x = q + (long)n * q_sn + (long)h * q_sh;
    const float4 u = ld4(x + i), w = ld4(x + i + half), f = ld4(inv_freq + i);
    float4 sn, cs;
    sincosf((float)p * f.x, &sn.x, &cs.x); sincosf((float)p * f.y, &sn.y, &cs.y);
    sincosf((float)p * f.z, &sn.z, &cs.z); sincosf((float)p * f.w, &sn.w, &cs.w);
    st4(x + i, make_float4(u.x * cs.x - w.x * sn.x, u.y * cs.y - w.y * sn.y, u.z * cs.z - w.z * sn.z, u.w * cs.w - w.w * sn.w));
    st4(x + i + half, make_float4(w.x * cs.x + u.x * sn.x, w.y * cs.y + u.y * sn.y, w.z * cs.z + u.z * sn.z, w.w * cs.w + u.w * sn.w));
}

template <typename T, int MAXE>
__global__ void latent_window_attn_kernel(const T* __restrict__ qa, long qa_sn, long qa_sh, const T* __restrict__ qr, long qr_sn,
                                          long qr_sh, const T* __restrict__ keys, long key_sb, int ring,
                                          const int* __restrict__ key_index, const int* __restrict__ pos0,
                                          const int* __restrict__ lens, int S, int H, int C, int R, int window, float scale,
                                          T* __restrict__ out, long out_sn, long out_sh) {
    const int n = blockIdx.x, h = blockIdx.y * blockDim.y + threadIdx.y, lane = threadIdx.x;
    if (h >= H) return;
    const int b = n / S, t = n % S, CR = C + R;
    T* o = out + (long)n * out_sn + (long)h * out_sh;
    if (t >= min(lens[b], S)) {
        for (int c = lane; c < C; c += 32) stf(o + c, 0.f);
        return;
    }
    float qv[MAXE], acc[MAXE];
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
        const int d = e * 32 + lane;
        acc[e] = 0.f;
        qv[e] = d < C ? ldf(qa + (long)n * qa_sn + (long)h * qa_sh + d) : (d < CR ? ldf(qr + (long)n * qr_sn + (long)h * qr_sh + d - C) : 0.f);
    }
    const int p = pos0[b] + t, lo = max(0, p - window + 1);
    const T* base = keys + (long)(key_index ? key_index[b] : b) * key_sb;
    int slot = lo % ring;
    float m = -INFINITY, l = 0.f;
    for (int j = lo; j <= p; ++j) {
        const T* row = base + (long)slot * CR;
        if (++slot == ring) slot = 0;
        float kv[MAXE], part = 0.f;
#pragma unroll
        for (int e = 0; e < MAXE; ++e) {
            const int d = e * 32 + lane;
            kv[e] = d < CR ? ldf(row + d) : 0.f;
            part = fmaf(qv[e], kv[e], part);
        }
        const float sc = warp_sum(part) * scale;
        const float mn = fmaxf(m, sc), corr = expf(m - mn), pj = expf(sc - mn);
        l = l * corr + pj;
#pragma unroll
        for (int e = 0; e < MAXE; ++e) acc[e] = fmaf(pj, kv[e], acc[e] * corr);
        m = mn;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
        const int d = e * 32 + lane;
        if (d < C) stf(o + d, acc[e] * inv);
    }
}

// Softmax over the visible keys of score rows produced by block matrix products (float in, activation dtype out, zeros where masked).
//   band mode: rows are (sequence b, query block, token t in block, head); column kk of a row holds position
//              j = blk*Qb - (w_eff - 1) + kk of the same sequence; visible: 0 <= j <= i and j > i - window, i = blk*Qb + t.
//   ring mode: rows are (sequence b, head) of one new token at position p = pos0[b]; column kk is ring row kk, which holds position
//              j = p - ((p - kk) mod ring); visible: j >= 0 and p - j < window.
template <typename Tout, bool RING>
__global__ void window_softmax_kernel(const float* __restrict__ scores, long rows, int span, float scale, int H, int Qb, int nblk, int w_eff,
                                      int window, const int* __restrict__ pos0, const int* __restrict__ lens, Tout* __restrict__ out) {
    const long r = (long)blockIdx.x * blockDim.y + threadIdx.y;
    const int lane = threadIdx.x;
    if (r >= rows) return;
    const float* sr = scores + r * span;
    Tout* orow = out + r * span;
    int b, i, j0;
    if (RING) { b = (int)(r / H); i = pos0[b]; j0 = 0; }
    else {
        const int t = (int)((r / H) % Qb), blk = (int)((r / ((long)H * Qb)) % nblk);
        b = (int)(r / ((long)H * Qb * nblk));
        i = blk * Qb + t;
        j0 = blk * Qb - (w_eff - 1);
    }
    const bool live = RING ? lens[b] > 0 : i < lens[b];
    auto visible = [&](int kk) -> bool {
        if (RING) { int m = (i - kk) % span; if (m < 0) m += span; return i - m >= 0 && m < window; }
        const int j = j0 + kk;
        return j >= 0 && j <= i && j > i - window;
    };
    float mx = -INFINITY;
    if (live)
        for (int kk = lane; kk < span; kk += 32)
            if (visible(kk)) mx = fmaxf(mx, sr[kk] * scale);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    if (live)
        for (int kk = lane; kk < span; kk += 32)
            if (visible(kk)) sum += expf(sr[kk] * scale - mx);
    sum = warp_sum(sum);
    const float inv = live ? 1.f / sum : 0.f;
    for (int kk = lane; kk < span; kk += 32) stf(orow + kk, (live && visible(kk)) ? expf(sr[kk] * scale - mx) * inv : 0.f);
}

void window_softmax(const float* scores, long rows, int span, float scale, int ring_mode, int H, int Qb, int nblk, int w_eff, int window,
                    const int* pos0, const int* lens, void* out, int out_bf16, cudaStream_t s) {
    if (rows == 0) return;
    dim3 block(32, 8), grid((unsigned)((rows + 7) / 8));
#define SEQMIX_SM(T, R) window_softmax_kernel<T, R><<<grid, block, 0, s>>>(scores, rows, span, scale, H, Qb, nblk, w_eff, window, pos0, lens, (T*)out)
    if (out_bf16) { if (ring_mode) SEQMIX_SM(bf16, true); else SEQMIX_SM(bf16, false); }
    else { if (ring_mode) SEQMIX_SM(float, true); else SEQMIX_SM(float, false); }
#undef SEQMIX_SM
}

void latent_kv_store(const void* kv, int bf, long kv_sb, long kv_st, int B, int S, int C, int R, int dims, const float* nw, float eps,
                     const float* inv_freq, const int* pos0, const int* lens, const int* slots, void* cache, int ring, void* rows,
                     cudaStream_t s) {
    dim3 block(32, 8), grid((B * S + 7) / 8);
    const size_t es = bf ? 2 : 4;
    auto al = [&](const void* p) { return p == nullptr || (uintptr_t)p % (4 * es) == 0; };
    const bool vec = C % 4 == 0 && R % 4 == 0 && dims % 8 == 0 && C <= kStoreVec * 128 && kv_sb % 4 == 0 && kv_st % 4 == 0 && al(kv) &&
                     al(cache) && al(rows) && (uintptr_t)nw % 16 == 0 && (uintptr_t)inv_freq % 16 == 0;
    if (vec) {
        if (bf) latent_kv_store_vec_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)kv, kv_sb, kv_st, B, S, C, R, dims, nw, eps, inv_freq,
                                                                       pos0, lens, slots, (bf16*)cache, ring, (bf16*)rows);
        else latent_kv_store_vec_kernel<float><<<grid, block, 0, s>>>((const float*)kv, kv_sb, kv_st, B, S, C, R, dims, nw, eps, inv_freq,
                                                                      pos0, lens, slots, (float*)cache, ring, (float*)rows);
        return;
    }
    if (bf) latent_kv_store_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)kv, kv_sb, kv_st, B, S, C, R, dims, nw, eps, inv_freq, pos0,
                                                               lens, slots, (bf16*)cache, ring, (bf16*)rows);
    else latent_kv_store_kernel<float><<<grid, block, 0, s>>>((const float*)kv, kv_sb, kv_st, B, S, C, R, dims, nw, eps, inv_freq, pos0,
                                                              lens, slots, (float*)cache, ring, (float*)rows);
}

void rope_q(void* q, int bf, long q_sn, long q_sh, int N, int S, int H, int dims, const float* inv_freq, const int* pos0, cudaStream_t s) {
    const long total = (long)N * H * (dims / 2);
    if (total == 0) return;
    const int threads = 256;
    const size_t es = bf ? 2 : 4;
    if (dims % 8 == 0 && q_sn % 4 == 0 && q_sh % 4 == 0 && (uintptr_t)q % (4 * es) == 0 && (uintptr_t)inv_freq % 16 == 0) {
        const unsigned vblocks = (unsigned)((total / 4 + threads - 1) / threads);
        if (bf) rope_q_vec_kernel<bf16><<<vblocks, threads, 0, s>>>((bf16*)q, q_sn, q_sh, N, S, H, dims, inv_freq, pos0);
        else rope_q_vec_kernel<float><<<vblocks, threads, 0, s>>>((float*)q, q_sn, q_sh, N, S, H, dims, inv_freq, pos0);
        return;
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (bf) rope_q_kernel<bf16><<<blocks, threads, 0, s>>>((bf16*)q, q_sn, q_sh, N, S, H, dims, inv_freq, pos0);
    else rope_q_kernel<float><<<blocks, threads, 0, s>>>((float*)q, q_sn, q_sh, N, S, H, dims, inv_freq, pos0);
}

template <typename T>
static void attn_launch(const void* qa, long qa_sn, long qa_sh, const void* qr, long qr_sn, long qr_sh, const void* keys, long key_sb,
                        int ring, const int* key_index, const int* pos0, const int* lens, int B, int S, int H, int C, int R, int window,
                        float scale, void* out, long out_sn, long out_sh, cudaStream_t s) {
    const int hb = H < 8 ? H : 8;
    dim3 block(32, hb), grid(B * S, (H + hb - 1) / hb);
    const int ne = (C + R + 31) / 32;
#define SEQMIX_ATTN(E)                                                                                                              \
    latent_window_attn_kernel<T, E><<<grid, block, 0, s>>>((const T*)qa, qa_sn, qa_sh, (const T*)qr, qr_sn, qr_sh, (const T*)keys, key_sb, \
                                                           ring, key_index, pos0, lens, S, H, C, R, window, scale, (T*)out, out_sn, out_sh)
    if (ne <= 3) SEQMIX_ATTN(3);
    else if (ne <= 6) SEQMIX_ATTN(6);
    else if (ne <= 10) SEQMIX_ATTN(10);
    else SEQMIX_ATTN(20);
#undef SEQMIX_ATTN
}

void latent_window_attention(const void* qa, int bf, long qa_sn, long qa_sh, const void* qr, long qr_sn, long qr_sh, const void* keys,
                             long key_sb, int ring, const int* key_index, const int* pos0, const int* lens, int B, int S, int H, int C,
                             int R, int window, float scale, void* out, long out_sn, long out_sh, cudaStream_t s) {
    if (bf) attn_launch<bf16>(qa, qa_sn, qa_sh, qr, qr_sn, qr_sh, keys, key_sb, ring, key_index, pos0, lens, B, S, H, C, R, window, scale, out, out_sn, out_sh, s);
    else attn_launch<float>(qa, qa_sn, qa_sh, qr, qr_sn, qr_sh, keys, key_sb, ring, key_index, pos0, lens, B, S, H, C, R, window, scale, out, out_sn, out_sh, s);
}

}  // namespace seqmix
