// Python bindings of the sequence-mixer kernels: shape / dtype / device checks, then the launchers of seqmix.h on the current stream.
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

// x [B,S,C] (last dim contiguous), w [C,taps], state [slots, taps-1, C] of x's dtype → out [B,S,C] of `out_bf16`'s dtype
Tensor short_conv(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, Tensor state, const Tensor& slots,
                  const Tensor& lens, bool fresh, bool residual, bool out_bf16) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.stride(2) == 1, "x must be [B,S,C] with a contiguous last dimension");
    const int B = x.size(0), S = x.size(1), C = x.size(2), taps = w.size(1);
    TORCH_CHECK(w.size(0) == C && taps >= 1 && taps <= 16, "taps must be 1..16");
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == x.scalar_type() && state.size(1) == taps - 1 && state.size(2) == C,
                "history must be [slots, taps-1, C] of the input's dtype");
    Tensor out = at::empty({B, S, C}, x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
    seqmix::short_conv(x.data_ptr(), is_bf(x), x.stride(0), x.stride(1), f32(w), bias ? f32(*bias) : nullptr, state.data_ptr(),
                       i32(slots), i32(lens), B, S, C, taps, fresh, residual, out.data_ptr(), out_bf16, stream());
    check_launch();
    return out;
}

// rows of x ([rows, C], row stride free) → out [rows, C] contiguous; w float [C] or one number
Tensor rms_norm(const Tensor& x, const Tensor& w, double eps, const c10::optional<Tensor>& gate, bool out_bf16) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "x must be [rows, C] with a contiguous last dimension");
    const int rows = x.size(0), C = x.size(1);
    TORCH_CHECK(w.numel() == 1 || w.numel() == C, "weight must hold 1 or C numbers");
    Tensor out = at::empty({rows, C}, x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
    const void* g = nullptr;
    long gs = 0;
    if (gate) {
        TORCH_CHECK(gate->scalar_type() == out.scalar_type() && gate->dim() == 2 && gate->stride(1) == 1, "gate must match the output");
        g = gate->data_ptr();
        gs = gate->stride(0);
    }
    if (rows)
        seqmix::rms_norm(x.data_ptr(), is_bf(x), x.stride(0), rows, C, f32(w), w.numel() == 1 ? 0 : 1, (float)eps, g, gs, out.data_ptr(),
                         out_bf16, C, nullptr, 0, stream());
    check_launch();
    return out;
}

// res [rows, C] float += norm(y) * w
void add_rms_norm_(Tensor res, const Tensor& y, const Tensor& w, double eps) {
    TORCH_CHECK(y.is_cuda() && y.dim() == 2 && y.stride(1) == 1 && res.dim() == 2 && res.stride(1) == 1 && res.scalar_type() == at::kFloat,
                "res must be float [rows, C], y [rows, C]");
    const int rows = y.size(0), C = y.size(1);
    TORCH_CHECK(res.size(0) == rows && res.size(1) == C && (w.numel() == 1 || w.numel() == C), "shape mismatch");
    if (rows)
        seqmix::rms_norm(y.data_ptr(), is_bf(y), y.stride(0), rows, C, f32(w), w.numel() == 1 ? 0 : 1, (float)eps, nullptr, 0, nullptr, 0, 0,
                         res.data_ptr<float>(), res.stride(0), stream());
    check_launch();
}

// kv [B,S,C+R] raw down-projection → normalised latent + rotated shared key, returned as rows [B,S,C+R] (if want_rows) and appended to
// cache [slots, ring, C+R] (if given)
Tensor latent_kv_store(const Tensor& kv, const Tensor& nw, double eps, const Tensor& inv_freq, int64_t dims, const Tensor& pos0,
                       const Tensor& lens, const Tensor& slots, const c10::optional<Tensor>& cache, bool want_rows) {
    TORCH_CHECK(kv.is_cuda() && kv.dim() == 3 && kv.stride(2) == 1, "kv must be [B,S,C+R]");
    const int B = kv.size(0), S = kv.size(1), C = nw.numel(), R = kv.size(2) - C;
    TORCH_CHECK(R >= 0 && dims % 2 == 0 && dims <= R && inv_freq.numel() == dims / 2, "bad rotary sizes");
    Tensor rows = want_rows ? at::zeros({B, S, C + R}, kv.options()) : Tensor();
    void* cp = nullptr;
    int ring = 1;
    if (cache) {
        TORCH_CHECK(cache->is_contiguous() && cache->scalar_type() == kv.scalar_type() && cache->size(2) == C + R, "bad cache");
        cp = cache->data_ptr();
        ring = cache->size(1);
    }
    seqmix::latent_kv_store(kv.data_ptr(), is_bf(kv), kv.stride(0), kv.stride(1), B, S, C, R, (int)dims, f32(nw), (float)eps, f32(inv_freq),
                            i32(pos0), i32(lens), i32(slots), cp, ring, want_rows ? rows.data_ptr() : nullptr, stream());
    check_launch();
    return rows;
}

// q [B,S,H,Dq]: rotate coordinates [off, off+dims) of every head in place
void rope_q_(Tensor q, int64_t off, int64_t dims, const Tensor& inv_freq, const Tensor& pos0) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && q.is_contiguous() && off + dims <= q.size(3) && inv_freq.numel() == dims / 2, "bad q");
    const int B = q.size(0), S = q.size(1), H = q.size(2), Dq = q.size(3);
    char* p = (char*)q.data_ptr() + off * q.element_size();
    seqmix::rope_q(p, is_bf(q), (long)H * Dq, Dq, B * S, S, H, (int)dims, f32(inv_freq), i32(pos0), stream());
    check_launch();
}

// qa [H, N, C] (absorbed queries, N = B*S), q [B,S,H,Dq] with the rotated part at `off`; keys [blocks, ring, C+R];
// key_index [B] (block of each sequence) or none (block b) → out [H, N, C]
Tensor latent_window_attention(const Tensor& qa, const Tensor& q, int64_t off, const Tensor& keys, const c10::optional<Tensor>& key_index,
                               const Tensor& pos0, const Tensor& lens, int64_t window, double scale) {
    TORCH_CHECK(qa.is_cuda() && qa.dim() == 3 && qa.is_contiguous() && q.dim() == 4 && q.is_contiguous() && keys.dim() == 3 && keys.is_contiguous(),
                "bad attention operands");
    const int H = qa.size(0), N = qa.size(1), C = qa.size(2), B = q.size(0), S = q.size(1), Dq = q.size(3), R = keys.size(2) - C;
    TORCH_CHECK(N == B * S && q.size(2) == H && R >= 0 && off + R <= Dq && C + R <= 640, "bad attention sizes (C + R <= 640)");
    TORCH_CHECK(qa.scalar_type() == q.scalar_type() && q.scalar_type() == keys.scalar_type(), "dtype mismatch");
    Tensor out = at::empty({H, N, C}, qa.options());
    const char* qr = (const char*)q.data_ptr() + off * q.element_size();
    if (S == 1 && seqmix::latent_ring_decode_fits(C, R)) {      // single tokens: split over the ring, partial softmaxes merged
        const long ns = seqmix::latent_ring_decode_splits((int)keys.size(1));
        const auto f = qa.options().dtype(at::kFloat);
        Tensor pm = at::empty({B, ns, H}, f), pl = at::empty({B, ns, H}, f), pa = at::empty({B, ns, H, C}, f);
        seqmix::latent_ring_decode(qa.data_ptr(), is_bf(qa), C, (long)N * C, qr, (long)H * Dq, Dq, keys.data_ptr(), keys.stride(0),
                                   (int)keys.size(1), key_index ? i32(*key_index) : nullptr, i32(pos0), i32(lens), B, H, C, R, (int)window,
                                   (float)scale, pm.data_ptr<float>(), pl.data_ptr<float>(), pa.data_ptr<float>(), out.data_ptr(), C,
                                   (long)N * C, stream());
        check_launch();
        return out;
    }
    seqmix::latent_window_attention(qa.data_ptr(), is_bf(qa), C, (long)N * C, qr, (long)H * Dq, Dq, keys.data_ptr(), keys.stride(0),
                                    (int)keys.size(1), key_index ? i32(*key_index) : nullptr, i32(pos0), i32(lens), B, S, H, C, R,
                                    (int)window, (float)scale, out.data_ptr(), C, (long)N * C, stream());
    check_launch();
    return out;
}

bool latent_prompt_attention_fits(int64_t D, int64_t R, int64_t CR, int64_t VD) {
    return seqmix::latent_prompt_attention_fits((int)D, (int)R, (int)CR, (int)VD);
}

// q [B,S,H,D+R], kx [B,S,H*D], rows [B,S,CR], v [B,S,H*VD] (all bfloat16, contiguous) → [B*S, H*VD]
Tensor latent_prompt_attention(const Tensor& q, const Tensor& kx, const Tensor& rows, const Tensor& v, const Tensor& lens, int64_t D,
                               int64_t R, int64_t VD, int64_t window, double scale) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && q.is_contiguous() && kx.is_contiguous() && rows.is_contiguous() && v.is_contiguous() &&
                    rows.dim() == 3, "bad prompt attention operands");
    TORCH_CHECK(is_bf(q) && is_bf(kx) && is_bf(rows) && is_bf(v), "the fused prompt attention takes bfloat16");
    const int B = q.size(0), S = q.size(1), H = q.size(2), CR = rows.size(2);
    TORCH_CHECK(q.size(3) == D + R && kx.numel() == (long)B * S * H * D && v.numel() == (long)B * S * H * VD && rows.size(0) == B &&
                    rows.size(1) == S && CR >= R, "shape mismatch");
    Tensor out = at::empty({(long)B * S, (long)H * VD}, q.options());
    bool ok = seqmix::latent_prompt_attention(q.data_ptr(), kx.data_ptr(), rows.data_ptr(), v.data_ptr(), i32(lens), B, S, H, (int)D, (int)R,
                                              CR, (int)VD, (int)window, (float)scale, out.data_ptr(), stream());
    TORCH_CHECK(ok, "latent_prompt_attention: sizes do not fit the kernel");
    check_launch();
    return out;
}

// scores float [..., span] (contiguous) → softmax over the visible keys, in `out_bf16`'s dtype.  Band mode: rows (b, block, t, head);
// ring mode: rows (b, head) of single tokens at positions pos0.
Tensor window_softmax(const Tensor& scores, double scale, bool ring_mode, int64_t H, int64_t Qb, int64_t nblk, int64_t w_eff, int64_t window,
                      const Tensor& pos0, const Tensor& lens, bool out_bf16) {
    TORCH_CHECK(scores.is_cuda() && scores.is_contiguous() && scores.scalar_type() == at::kFloat, "scores must be contiguous float");
    const int span = scores.size(-1);
    const long rows = scores.numel() / span;
    Tensor out = at::empty(scores.sizes(), scores.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
    seqmix::window_softmax(scores.data_ptr<float>(), rows, span, (float)scale, ring_mode, (int)H, (int)Qb, (int)nblk, (int)w_eff, (int)window,
                           i32(pos0), i32(lens), out.data_ptr(), out_bf16, stream());
    check_launch();
    return out;
}

// q,k [B,S,H,D], v [B,S,H,V] (views with equal batch / token strides), z [B,S,H*D] → o float [B,S,H,V]; state [slots,H,D,V] float
// Runs of at least this many tokens take the chunked form (matrix products); shorter ones and single tokens the token by token scan.
static const int kGlaChunkedFrom = 32;

// Float matrix products stay true float here whatever the process-wide setting is: they carry the recurrence.
struct FloatProducts {
    bool was;
    FloatProducts() : was(at::globalContext().allowTF32CuBLAS()) { at::globalContext().setAllowTF32CuBLAS(false); }
    ~FloatProducts() { at::globalContext().setAllowTF32CuBLAS(was); }
};

static Tensor gla_scan_chunked(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& z, const Tensor& zbias, double tau,
                               Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), V = v.size(3), C = seqmix::gla_chunk_tokens();
    const auto f = q.options().dtype(at::kFloat);
    const long es = q.element_size();
    // the states before every chunk are materialised ([chunks, D, V] floats per head): long prompts go segment by segment
    const long per_chunk = (long)B * H * D * V * 4;
    const long seg_chunks = std::max<long>(1, (1L << 30) / per_chunk);
    const long seg = seg_chunks * C;
    Tensor out = at::empty({B, S, H, V}, f);
    FloatProducts guard;
    for (long s0 = 0; s0 < S; s0 += seg) {
        const int Sg = (int)std::min<long>(seg, S - s0), nC = (Sg + C - 1) / C;
        const long n = (long)B * H * nC;
        Tensor lens_g = s0 == 0 ? lens : (lens - (int)s0).clamp_min(0).to(at::kInt).contiguous();
        Tensor Qe = at::empty({n, C, D}, f), Ke = at::empty({n, C, D}, f), Bc = at::empty({n, C, D}, f), G = at::empty({n, D}, f);
        Tensor Vf = at::empty({n, C, V}, f), A = at::empty({n, C, C}, f);
        const char *qp = (const char*)q.data_ptr() + s0 * q.stride(1) * es, *kp = (const char*)k.data_ptr() + s0 * k.stride(1) * es;
        const char *vp = (const char*)v.data_ptr() + s0 * v.stride(1) * es, *zp = (const char*)z.data_ptr() + s0 * z.stride(1) * es;
        seqmix::gla_chunk_prep(qp, kp, vp, is_bf(q), q.stride(0), q.stride(1), zp, z.stride(0), z.stride(1), f32(zbias), (float)(1.0 / tau),
                               (float)(1.0 / std::sqrt((double)D)), i32(lens_g), B, Sg, H, D, V, nC, Qe.data_ptr<float>(),
                               Ke.data_ptr<float>(), Bc.data_ptr<float>(), G.data_ptr<float>(), Vf.data_ptr<float>(), A.data_ptr<float>(),
                               stream());
        check_launch();
        Tensor Sl = at::bmm(Ke.transpose(1, 2), Vf);                                             // [n, D, V]
        seqmix::gla_carry(Sl.data_ptr<float>(), G.data_ptr<float>(), state.data_ptr<float>(), i32(slots), fresh && s0 == 0, B, nC, H, D, V,
                          stream());
        check_launch();
        Tensor O = at::baddbmm(at::bmm(A, Vf), Qe, Sl);                                          // [n, C, V]
        out.slice(1, s0, s0 + Sg).copy_(O.view({B, H, (long)nC * C, V}).slice(2, 0, Sg).permute({0, 2, 1, 3}));
    }
    return out;
}

Tensor gla_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& z, const Tensor& zbias, double tau, Tensor state,
                const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && v.dim() == 4 && q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && z.stride(2) == 1,
                "bad recurrence operands");
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), V = v.size(3);
    TORCH_CHECK(H == 1 || (q.stride(2) == D && k.stride(2) == D && v.stride(2) == V), "heads must be laid out one after another");
    TORCH_CHECK((B == 1 || (q.stride(0) == k.stride(0) && q.stride(0) == v.stride(0))) &&
                    (S == 1 || (q.stride(1) == k.stride(1) && q.stride(1) == v.stride(1))),
                "q, k, v must share their batch and token strides");   // a stride of a dimension of size 1 is never used
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.size(1) == H && state.size(2) == D && state.size(3) == V,
                "state must be float [slots,H,D,V]");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type() && q.scalar_type() == z.scalar_type(), "dtype mismatch");
    if (S >= kGlaChunkedFrom) return gla_scan_chunked(q, k, v, z, zbias, tau, state, slots, lens, fresh);
    Tensor out = at::empty({B, S, H, V}, q.options().dtype(at::kFloat));
    if (S == 1 && seqmix::gla_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), is_bf(q), q.stride(0), z.data_ptr(), z.stride(0), f32(zbias),
                                   (float)(1.0 / tau), (float)(1.0 / std::sqrt((double)D)), state.data_ptr<float>(), i32(slots), i32(lens),
                                   fresh, B, H, D, V, out.data_ptr<float>(), stream())) {
        check_launch();
        return out;
    }
    bool ok = seqmix::gla_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), is_bf(q), q.stride(0), q.stride(1), z.data_ptr(), z.stride(0),
                               z.stride(1), f32(zbias), (float)(1.0 / tau), (float)(1.0 / std::sqrt((double)D)), state.data_ptr<float>(),
                               i32(slots), i32(lens), fresh, B, S, H, D, V, out.data_ptr<float>(), stream());
    TORCH_CHECK(ok, "gla_scan: no launch shape for key size ", D, " and value size ", V);
    check_launch();
    return out;
}

// u [B,S,W] contiguous, gr / gi float [blocks, B*S, W/blocks], y [B,S,W] view (pre-activation) → out [B,S,W]; state [slots, W] float
Tensor rglru_scan(const Tensor& u, const Tensor& gr, const Tensor& gi, const Tensor& rbias, const Tensor& ibias, const Tensor& lam_sp,
                  const Tensor& y, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(u.is_cuda() && u.dim() == 3 && u.is_contiguous() && y.dim() == 3 && y.stride(2) == 1 && gr.dim() == 3, "bad operands");
    const int B = u.size(0), S = u.size(1), W = u.size(2), wb = gr.size(2);
    TORCH_CHECK(gr.size(0) * wb == W && gr.size(1) == (long)B * S && gi.sizes() == gr.sizes() && u.scalar_type() == y.scalar_type(), "bad gates");
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.size(1) == W, "state must be float [slots, W]");
    Tensor out = at::empty({B, S, W}, u.options());
    seqmix::rglru_scan(u.data_ptr(), is_bf(u), f32(gr), f32(gi), wb, f32(rbias), f32(ibias), f32(lam_sp), y.data_ptr(), y.stride(0), y.stride(1),
                       state.data_ptr<float>(), i32(slots), i32(lens), fresh, B, S, W, out.data_ptr(), stream());
    check_launch();
    return out;
}

Tensor xielu(const Tensor& x, double ap, double an) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be contiguous");
    Tensor out = at::empty_like(x);
    seqmix::xielu(x.data_ptr(), out.data_ptr(), is_bf(x), x.numel(), (float)ap, (float)an, stream());
    check_launch();
    return out;
}

Tensor gelu_erf(const Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be contiguous");
    Tensor out = at::empty_like(x);
    seqmix::gelu_erf(x.data_ptr(), out.data_ptr(), is_bf(x), x.numel(), stream());
    check_launch();
    return out;
}

// w [E,O,I], sel int [M], x [M,I] → act(w[sel[m]] x[m]) [M,O]
Tensor indexed_gemv(const Tensor& w, const Tensor& sel, const Tensor& x, bool gelu) {
    TORCH_CHECK(w.is_cuda() && w.dim() == 3 && w.is_contiguous() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == w.scalar_type(), "bad gemv operands");
    const int M = x.size(0), O = w.size(1), I = w.size(2);
    TORCH_CHECK(x.size(1) == I && sel.numel() == M, "shape mismatch");
    Tensor out = at::empty({M, O}, x.options());
    seqmix::indexed_gemv(w.data_ptr(), i32(sel), x.data_ptr(), is_bf(x), x.stride(0), M, O, I, gelu, out.data_ptr(), stream());
    check_launch();
    return out;
}

// rows [M,C], src int [N,top], weight float [N,top], base [N,C] or none → [N,C]
Tensor moe_combine(const Tensor& rows, const Tensor& src, const Tensor& weight, const c10::optional<Tensor>& base) {
    TORCH_CHECK(rows.is_cuda() && rows.dim() == 2 && rows.is_contiguous() && src.dim() == 2, "bad combine operands");
    const int N = src.size(0), top = src.size(1), C = rows.size(1);
    if (base) TORCH_CHECK(base->is_contiguous() && base->scalar_type() == rows.scalar_type() && base->size(0) == N && base->size(1) == C, "bad base");
    Tensor out = at::empty({N, C}, rows.options());
    seqmix::moe_combine(rows.data_ptr(), i32(src), f32(weight), base ? base->data_ptr() : nullptr, is_bf(rows), N, top, C, out.data_ptr(), stream());
    check_launch();
    return out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("short_conv", &short_conv);
    m.def("rms_norm", &rms_norm);
    m.def("add_rms_norm_", &add_rms_norm_);
    m.def("latent_kv_store", &latent_kv_store);
    m.def("rope_q_", &rope_q_);
    m.def("latent_window_attention", &latent_window_attention);
    m.def("window_softmax", &window_softmax);
    m.def("latent_prompt_attention", &latent_prompt_attention);
    m.def("latent_prompt_attention_fits", &latent_prompt_attention_fits);
    m.def("gla_scan", &gla_scan);
    m.def("rglru_scan", &rglru_scan);
    m.def("xielu", &xielu);
    m.def("gelu_erf", &gelu_erf);
    m.def("indexed_gemv", &indexed_gemv);
    m.def("moe_combine", &moe_combine);
}
