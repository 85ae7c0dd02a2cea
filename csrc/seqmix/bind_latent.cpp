// Python bindings of the latent sliding-window attention kernels.
#include "bind_common.h"

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

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("latent_kv_store", &latent_kv_store);
    m.def("rope_q_", &rope_q_);
    m.def("latent_window_attention", &latent_window_attention);
    m.def("window_softmax", &window_softmax);
    m.def("latent_prompt_attention", &latent_prompt_attention);
    m.def("latent_prompt_attention_fits", &latent_prompt_attention_fits);
}
