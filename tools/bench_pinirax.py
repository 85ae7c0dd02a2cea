"""``bench.py --mode pinirax``: serving throughput of the Pinirax design at layer sizes that resemble a real model (random weights),
beside the framework's closest existing model — Naguzen, the other family of window attention + gated recurrences + routed
feed-forwards on the slot-based serving path — at equal width and depth; plus every kernel the design added, timed alone against the
measured copy bandwidth / GEMM throughput, beside the like kernel of the Naguzen path.  One GPU, bfloat16.  Device time (CUDA
events), >= 3 warm-up iterations; the weights of either model (> 1 GB) exceed L2, and the kernel timings flush L2 (a 512 MiB write)
between iterations; every kernel row is replayed from a CUDA graph.

Layers (width 2048): parallel [window attention 16 heads / 4 KV heads of 128, value 128, window 1024, cap 30 | delta rule 16 value
heads of 128 over 4 q/k heads of 128, 4 taps] + routed | state space 32 heads of 128, state 128, 4 taps + routed | parallel + routed |
state space + routed; routed: 32 experts of ff 1024 (gated), top 4, 4 identity experts."""
from __future__ import annotations

import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tools"))

import bench_naguzen as base  # noqa: E402

WIDTH, VOCAB = base.WIDTH, base.VOCAB


def pinirax_layers():
    moe = {"kind": "moe", "expert": {"ff": 1024}, "router": {"experts": 32, "identity": 4, "top": 4}}
    par = {"type": "parallel", "mlp": moe,
           "mixer": {"left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 1.0 / math.sqrt(128), "softcap": 30.0},
                     "right": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "conv": 4}, "left_scale": 0.8, "right_scale": 0.9}}
    ssm = {"type": "mamba2", "mlp": moe, "mixer": {"heads": 32, "vdim": 128, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}}
    return [par, ssm, par, ssm]


def build_pinirax(dev, batch, max_len):
    import torch

    from neuronx_distributed_b200.models.pinirax import PiniraxConfig, PiniraxForInference

    cfg = PiniraxConfig(vocab=VOCAB, width=WIDTH, layers=pinirax_layers(), norm_eps=1e-6, embedding_scale=8.0, dtype=torch.bfloat16, device=dev)
    m = PiniraxForInference(cfg, batch_size=batch, max_seq_len=max_len).eval()
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dtype == torch.bfloat16 or "router" in name:
                p.normal_(0.0, 0.02 if p.dim() > 1 else 0.0, generator=g)
                if "router" in name:                       # as a checkpoint stored in bfloat16 would hold it
                    p.copy_(p.to(torch.bfloat16).float())
            elif "conv.weight" in name:
                p.normal_(0.0, 0.2, generator=g)
            elif name.endswith(("a_log",)):
                p.fill_(-1.0)
            elif name.endswith(("q_norm", "k_norm", "mixer.norm", "right.norm", "d_skip")):
                p.fill_(1.0)
        m.lm.embed.normal_(0.0, 1.0, generator=g)
    return m


def kernel_table(dev, steps, warmup):
    """Each new kernel alone at the sizes of the model above (4 x 2048 prompt tokens; 8 decoding rows) → time, achieved GB/s or
    TFLOP/s, fraction of the measured peak; the like kernel of the Naguzen path is timed the same way in the row after it."""
    import torch

    from neuronx_distributed_b200.ops import seqmix

    hbm, tfl, src = base._peaks()
    flush = torch.empty(128 << 20, dtype=torch.float32, device=dev)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    B, S, W = 4, 2048, WIDTH
    N = B * S
    rnd = lambda *s, dtype=bf: torch.randn(*s, device=dev, dtype=f32).to(dtype)
    lens, slots, pos0 = torch.full((B,), S, dtype=i32, device=dev), torch.arange(B, dtype=i32, device=dev), torch.zeros(B, dtype=i32, device=dev)
    rows = []

    def replayed(fn):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g.replay
        except Exception:
            torch.cuda.synchronize()
            return fn

    def add(name, fn, bytes_=0, flops=0, like=None):
        ms = base._timed(replayed(fn), steps, warmup, flush)
        r = {"kernel": name, "ms": round(ms, 4)}
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
            r["frac_bf16_gemm"] = round(flops / ms / 1e9 / tfl, 4)
        if like:
            r["like_of"] = like
        rows.append(r)

    # embedding, norms, convolution
    table, toks = rnd(VOCAB, W), torch.randint(0, VOCAB, (B, S), device=dev)
    inv = seqmix.sinusoid_inv_freq(W, 10000.0, dev)
    add("embed_sinusoid -> f32 stream", lambda: seqmix.embed_sinusoid(toks, table, 8.0, inv, pos0), N * W * 6)
    I = 4096
    y32, z16, wI = rnd(N, I, dtype=f32), rnd(N, I), torch.ones(I, device=dev)
    add("group_rms_norm_gated (gate first, 1 group of 4096)", lambda: seqmix.group_rms_norm_gated(y32, z16, wI, 1, 1e-6, True, out_dtype=bf), N * I * 8)
    w128 = torch.ones(128, device=dev)
    add("group_rms_norm_gated (16 heads of 128, gate after)", lambda: seqmix.group_rms_norm_gated(y32[:, :2048], z16[:, :2048], w128, 16, 1e-6, False, out_dtype=bf),
        N * 2048 * 8)
    add("naguzen rms_norm f32->bf16 with silu gate (rows of 512)", lambda: seqmix.rms_norm(y32.view(N * 8, 512), torch.ones(512, device=dev), 1e-6, gate=z16.view(N * 8, 512), out_dtype=bf),
        N * I * 8, like="group_rms_norm_gated")
    C = 4096 + 256
    xc, cw, cb = rnd(B, S, C), rnd(C, 4, dtype=f32), torch.zeros(C, device=dev)
    stc = torch.zeros(B, 3, C, dtype=bf, device=dev)
    add("short_conv + bias + silu bf16 (4352 channels)", lambda: seqmix.short_conv(xc, cw, cb, stc, slots, lens, True, False, bf, True), N * C * 4)
    x32, st32 = rnd(B, S, W, dtype=f32), torch.zeros(B, 3, W, dtype=f32, device=dev)
    add("naguzen short_conv residual f32->bf16", lambda: seqmix.short_conv(x32, cw[:W].contiguous(), None, st32, slots, lens, True, True, bf), N * W * 6,
        like="short_conv + silu")
    # window attention
    H, G, D, V, win = 16, 4, 128, 128, 1024
    q, k, v, gate = rnd(B, S, H, D), rnd(B, S, G, D), rnd(B, S, G, V), rnd(B, S, H)
    qw = torch.ones(D, device=dev)
    kc, vc = torch.zeros(B, win, G, D, dtype=bf, device=dev), torch.zeros(B, win, G, V, dtype=bf, device=dev)
    add("window_qk_prepare (q/k head norms in place + ring store)", lambda: seqmix.window_qk_prepare(q, k, v, qw, qw, 1e-6, pos0, lens, slots, kc, vc),
        N * (H + G) * D * 4 + B * win * G * (D + V) * 4)
    Cl, R = 512, 64
    kvl, nw, invr = rnd(B, S, Cl + R), torch.ones(Cl, device=dev), seqmix.rotary_inv_freq(R, 10000.0, dev)
    cachel = torch.zeros(B, win, Cl + R, dtype=bf, device=dev)
    add("naguzen latent_kv_store (norm + rope + ring append)", lambda: seqmix.latent_kv_store(kvl, nw, 1e-6, invr, R, pos0, lens, slots, cachel, True),
        N * (Cl + R) * 4 + B * win * (Cl + R) * 2, like="window_qk_prepare")
    pairs = B * H * sum(min(p + 1, win) for p in range(S))
    out = torch.empty(N, H * V, dtype=bf, device=dev)
    add("window_attention_prompt (GQA 16/4 x 128, window 1024, cap, gate)", lambda: seqmix.window_attention_prompt(q, k, v, gate, lens, win, 0.088, 30.0, out, 0.8),
        flops=pairs * 2 * (D + V))
    ql, kx, vx = rnd(B, S, H, D + R), rnd(B, S, H * D), rnd(B, S, H * V)
    add("naguzen latent_prompt_attention (16 heads, 128+64 / 128, window 1024)", lambda: seqmix.latent_prompt_attention(ql, kx, kvl, vx, lens, D, R, V, win, 0.07),
        flops=pairs * 2 * (D + R + V), like="window_attention_prompt")
    Bd = 8
    q1, g1 = rnd(Bd, 1, H, D), rnd(Bd, 1, H)
    kc8, vc8 = rnd(Bd, win, G, D), rnd(Bd, win, G, V)
    l1, s8, p8 = torch.ones(Bd, dtype=i32, device=dev), torch.arange(Bd, dtype=i32, device=dev), torch.full((Bd,), 2047, dtype=i32, device=dev)
    o1 = torch.empty(Bd, H * V, dtype=bf, device=dev)
    add("window_attention_token (8 rows, ring 1024, 4 KV heads)", lambda: seqmix.window_attention_token(q1, kc8, vc8, g1, s8, p8, l1, win, 0.088, 30.0, o1, 0.8),
        bytes_=Bd * win * G * (D + V) * 2)
    qa1, q1l, cache8 = rnd(H, Bd, Cl), rnd(Bd, 1, H, D + R), rnd(Bd, win, Cl + R)
    add("naguzen latent attention decode (8 rows, ring 1024)", lambda: seqmix.latent_window_attention(qa1, q1l, D, cache8, s8, p8, l1, win, 0.07),
        bytes_=Bd * win * (Cl + R) * 2, like="window_attention_token")
    # recurrences
    Hd, Gd, Dd, Vd = 16, 4, 128, 128
    qd, kd, vd = rnd(B, S, Gd, Dd), rnd(B, S, Gd, Dd), rnd(B, S, Hd, Vd)
    ba = rnd(B, S, 2 * Hd, dtype=f32)
    al, db = torch.full((Hd,), -1.0, device=dev), torch.zeros(Hd, device=dev)
    std = torch.zeros(B, Hd, Dd, Vd, device=dev)
    add("gated_delta_scan prompt (16 heads, 128 x 128 state)", lambda: seqmix.gated_delta_scan(qd, kd, vd, ba[..., :Hd], ba[..., Hd:], al, db, std, slots, lens, True),
        bytes_=N * (2 * Gd * Dd * 2 + Hd * Vd * 2 + Hd * Vd * 4), flops=N * Hd * Dd * Vd * 6)
    Hs, Ns, Vs = 32, 128, 128
    xs, bs_, cs = rnd(B, S, Hs, Vs), rnd(B, S, 1, Ns), rnd(B, S, 1, Ns)
    dts = rnd(B, S, Hs, dtype=f32)
    als, dbs, dsk = torch.full((Hs,), -1.0, device=dev), torch.zeros(Hs, device=dev), torch.ones(Hs, device=dev)
    sts = torch.zeros(B, Hs, Ns, Vs, device=dev)
    add("ssd_scan prompt (32 heads, 128 x 128 state)", lambda: seqmix.ssd_scan(xs, bs_, cs, dts, als, dbs, dsk, sts, slots, lens, True),
        bytes_=N * (Hs * Vs * 2 + 2 * Ns * 2 + Hs * Vs * 4), flops=N * Hs * Ns * Vs * 4)
    Hg, Dg, Vg = 4, 256, 512
    p = rnd(B, S, 2 * Hg * Dg + Hg * Vg)
    qg, kg = p[..., :Hg * Dg].unflatten(-1, (Hg, Dg)), p[..., Hg * Dg:2 * Hg * Dg].unflatten(-1, (Hg, Dg))
    vg, z = p[..., 2 * Hg * Dg:].unflatten(-1, (Hg, Vg)), rnd(B, S, Hg * Dg)
    zb, stg = torch.full((Hg * Dg,), 3.0, device=dev), torch.zeros(B, Hg, Dg, Vg, device=dev)
    add("naguzen gla_scan prompt (4 heads, 256 x 512 state)", lambda: seqmix.gla_scan(qg, kg, vg, z, zb, 16.0, stg, slots, lens, True),
        bytes_=N * (3 * Hg * Dg * 2 + Hg * Vg * 2 + Hg * Vg * 4), flops=N * Hg * Dg * Vg * 4, like="gated_delta_scan / ssd_scan prompt")
    q1d, k1d, v1d, ba1 = rnd(Bd, 1, Gd, Dd), rnd(Bd, 1, Gd, Dd), rnd(Bd, 1, Hd, Vd), rnd(Bd, 1, 2 * Hd, dtype=f32)
    st8 = torch.zeros(Bd, Hd, Dd, Vd, device=dev)
    add("gated_delta_scan decode (8 rows)", lambda: seqmix.gated_delta_scan(q1d, k1d, v1d, ba1[..., :Hd], ba1[..., Hd:], al, db, st8, s8, l1, False),
        bytes_=Bd * Hd * Dd * Vd * 8)
    x1s, b1s, c1s, dt1 = rnd(Bd, 1, Hs, Vs), rnd(Bd, 1, 1, Ns), rnd(Bd, 1, 1, Ns), rnd(Bd, 1, Hs, dtype=f32)
    sts8 = torch.zeros(Bd, Hs, Ns, Vs, device=dev)
    add("ssd_scan decode (8 rows)", lambda: seqmix.ssd_scan(x1s, b1s, c1s, dt1, als, dbs, dsk, sts8, s8, l1, False), bytes_=Bd * Hs * Ns * Vs * 8)
    p1, z1, stg8 = rnd(Bd, 1, 2 * Hg * Dg + Hg * Vg), rnd(Bd, 1, Hg * Dg), torch.zeros(Bd, Hg, Dg, Vg, device=dev)
    q1g, k1g = p1[..., :Hg * Dg].unflatten(-1, (Hg, Dg)), p1[..., Hg * Dg:2 * Hg * Dg].unflatten(-1, (Hg, Dg))
    v1g = p1[..., 2 * Hg * Dg:].unflatten(-1, (Hg, Vg))
    add("naguzen gla_scan decode (8 rows)", lambda: seqmix.gla_scan(q1g, k1g, v1g, z1, zb, 16.0, stg8, s8, l1, False), bytes_=Bd * Hg * Dg * Vg * 8,
        like="gated_delta_scan / ssd_scan decode")
    # routed small batch
    E, ff, top = 32, 1024, 4
    wgu, wu, xe = rnd(E, 2 * ff, W), rnd(E, ff, W), rnd(Bd * top, W)
    sel = torch.randint(0, E, (Bd * top,), device=dev, dtype=i32)
    add("indexed_gemv gate|up + silu-glu (32 rows x expert [2048,2048])", lambda: seqmix.indexed_gemv(wgu, sel, xe, "silu_glu"), bytes_=Bd * top * 2 * ff * W * 2)
    add("naguzen indexed_gemv up + gelu (32 rows x expert [1024,2048])", lambda: seqmix.indexed_gemv(wu, sel, xe, "gelu"), bytes_=Bd * top * ff * W * 2,
        like="indexed_gemv silu-glu")
    gu = rnd(N, 2 * ff)
    add("silu_mul [N, 2x1024]", lambda: seqmix.silu_mul(gu), N * ff * 6)
    up = rnd(N, ff)
    add("naguzen gelu_erf [N,1024]", lambda: seqmix.gelu_erf(up), N * ff * 4, like="silu_mul")
    return {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "source": src}, "rows": rows}


def main(args) -> int:
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29538")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    from neuronx_distributed_b200.parallel_layers import parallel_state as ps

    ps.initialize_model_parallel(tensor_model_parallel_size=1)
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    out = {"mode": "pinirax", "dtype": "bf16", "data": "synthetic", "steps": steps, "warmup": warmup, "n_gpus": 1,
           "l2": "weights of either model exceed L2; kernel rows flush L2 between iterations"}
    shapes = [(4, 2048), (1, 8192), (8, 512)]
    for name, make in (("pinirax", build_pinirax), ("naguzen", base.build_naguzen)):
        res = []
        for B, S in shapes:
            model = make(dev, B, S + 64)
            res.append(base.throughput(model, dev, B, S, S, steps, warmup))
            del model
            torch.cuda.empty_cache()
        out[name] = res
    out["kernels"] = kernel_table(dev, max(steps, 5), warmup)
    print(json.dumps(out), flush=True)
    dist.destroy_process_group()
    return 0
