"""Pinirax serving path against the plain oracle (tests/pinirax_oracle.py): every mechanism alone, whole prompts, prompt + token by
token decoding, unequal batches, reused slots, window edges, far keys through the recurrent states, other sizes, greedy generation
through the serving entry points, the registry / checkpoint reader, the trace runner and the generation command line.
Configurations and weights are made here (random, seeded)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import pinirax_oracle as oracle  # noqa: E402

from neuronx_distributed_b200.inference.hf_adapter import HuggingFaceGenerationAdapter  # noqa: E402
from neuronx_distributed_b200.inference.state_cache import StepContext  # noqa: E402
from neuronx_distributed_b200.inference.trace_replay import TraceReplayer  # noqa: E402
from neuronx_distributed_b200.models import registry  # noqa: E402
from neuronx_distributed_b200.models.pinirax import PiniraxConfig, PiniraxForInference, complete_config, load_pinirax_weights  # noqa: E402
from neuronx_distributed_b200.modules.moe.routed_ffn import RoutedFFN  # noqa: E402
from neuronx_distributed_b200.ops import seqmix  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


# ------------------------------------------------------------------------------------------------------------------ model making
def left_spec(heads=4, kv_heads=2, dim=24, vdim=40, window=7, softcap=20.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": 1.0 / math.sqrt(dim),
            "softcap": softcap}


def right_spec(heads=4, kv_heads=2, dim=20, vdim=12, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def par(left=None, right=None, ls=0.7, rs=1.2, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left or left_spec(), "right": right or right_spec(), "left_scale": ls, "right_scale": rs}}


def ssm(heads=4, vdim=12, state=10, groups=2, norm_groups=2, conv=4, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}


def moe(experts=5, identity=2, top=3, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def make_cfg(layers, vocab=50, width=48, eps=1e-5, scale=3.0):
    return {"architecture": "Pinirax", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}


def random_checkpoint(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    bf = lambda t: t.to(torch.bfloat16).float()
    lin = lambda o, i, s=1.0: bf(torch.randn(o, i, generator=g) * s / math.sqrt(i))
    vec = lambda n, s=1.0, m=0.0: bf(torch.randn(n, generator=g) * s + m)
    W, w = cfg["width"], {}
    w["embed"], w["head"], w["final.norm"] = bf(torch.randn(cfg["vocab"], W, generator=g)), lin(cfg["vocab"], W), vec(W, 0.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b"):
            w[p + n] = vec(W, 0.2)
        if L["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            w.update({q + "q": lin(H * D, W, 2.0), q + "q.b": vec(H * D, 0.3), q + "k": lin(G * D, W, 2.0), q + "k.b": vec(G * D, 0.3),
                      q + "v": lin(G * V, W), q + "v.b": vec(G * V, 0.3), q + "q.norm": vec(D, 0.3, 1.5), q + "k.norm": vec(D, 0.3, 1.5),
                      q + "g": lin(H, W, 2.0), q + "o": lin(W, H * V)})
            H, G, D, V, taps = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            q = p + "mix.right."
            w.update({q + "q": lin(G * D, W, 2.0), q + "k": lin(G * D, W, 2.0), q + "v": lin(H * V, W, 2.0), q + "g": lin(H * V, W),
                      q + "q.conv": bf(torch.randn(G * D, taps, generator=g) * 0.6), q + "k.conv": bf(torch.randn(G * D, taps, generator=g) * 0.6),
                      q + "v.conv": bf(torch.randn(H * V, taps, generator=g) * 0.6), q + "b": lin(H, W, 2.0), q + "a": lin(H, W, 2.0),
                      q + "A_log": vec(H, 0.5, -1.0), q + "dt_bias": vec(H, 0.5), q + "norm": vec(V, 0.2, 1.0), q + "o": lin(W, H * V)})
        else:
            H, V, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, q = H * V, p + "mix."
            w.update({q + "in": lin(2 * inner + 2 * G * N + H, W, 2.0), q + "conv": bf(torch.randn(inner + 2 * G * N, taps, generator=g) * 0.6),
                      q + "conv.b": vec(inner + 2 * G * N, 0.2), q + "dt_bias": vec(H, 0.5), q + "A_log": vec(H, 0.5, -0.5), q + "D": vec(H, 0.5, 1.0),
                      q + "norm": vec(inner, 0.2, 1.0), q + "o": lin(W, inner)})
        f = L.get("mlp")
        if not f:
            continue
        for n in ("norm2", "norm2b"):
            w[p + n] = vec(W, 0.2)
        E, I = f["router"]["experts"], f["router"].get("identity", 0)
        for e in range(E):
            w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = lin(f["expert"]["ff"], W, 2.0), lin(f["expert"]["ff"], W)
            w[p + f"mlp.e{e}.down"] = lin(W, f["expert"]["ff"])
        w[p + "mlp.router"], w[p + "mlp.correction"] = lin(E + I, W, 3.0), vec(E + I, 0.3)
    return w


def build(cfg, weights, device, dtype=torch.float32, max_seq_len=4096, batch_size=1):
    full = complete_config(cfg, {k: tuple(v.shape) for k, v in weights.items()})
    m = PiniraxForInference(PiniraxConfig.from_dict(full, dtype=dtype, device=torch.device(device)), batch_size=batch_size,
                            max_seq_len=max_seq_len, on_device_sampling=False)
    load_pinirax_weights(m.lm, weights)
    return m.eval()


def tokens_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def run_alone(model, toks, prompt):
    """Prompt of ``prompt`` tokens in one step, the rest one by one → logits at every position [S, vocab] (float, cpu)."""
    mgr = model.states
    slot = mgr.alloc()
    dev = next(model.parameters()).device
    x = model.forward_step(torch.tensor([toks[:prompt]], device=dev), [prompt], [slot], [0], True)
    out = [model.logits(x[0])]
    for p in range(prompt, len(toks)):
        x = model.forward_step(torch.tensor([[toks[p]]], device=dev), [1], [slot], [p], False)
        out.append(model.logits(x[0]))
    mgr.free(slot)
    return torch.cat(out).cpu()


def close(got, want, tol):
    """Mean-free difference relative to the spread of the expected values, per position."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    ref = (want - want.mean(-1, keepdim=True)).double().pow(2).mean().sqrt()
    err = (d.pow(2).mean(-1).sqrt() / ref).max().item()
    assert err < tol, f"relative error {err:.3e} >= {tol}"


MIXED = [par(mlp=moe()), ssm(mlp=moe(experts=4, identity=0, top=1)), par(left_spec(heads=2, kv_heads=2, window=5), right_spec(heads=2, kv_heads=1, conv=2), mlp=None),
         ssm(heads=2, vdim=40, state=33, groups=1, norm_groups=1, conv=2, mlp=moe(experts=3, identity=3, top=2)), par(mlp=moe(top=5))]
TOL32 = 2e-4


def ctx_for(lens, slots, pos0, fresh, device):
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return StepContext(t(lens), t(slots), t(pos0), fresh)


# ------------------------------------------------------------------------------------------------------------ single mechanisms
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("W", [48, 37])
def test_embedding_with_sinusoids(device, W):
    g = torch.Generator().manual_seed(W)
    table = torch.randn(30, W, generator=g)
    toks = torch.randint(0, 30, (2, 9), generator=g)
    got = seqmix.embed_sinusoid(toks.to(device), table.to(device), 2.5, seqmix.sinusoid_inv_freq(W, 10000.0, device),
                                torch.tensor([0, 700], dtype=torch.int32, device=device)).cpu()
    for b, p0 in enumerate((0, 700)):
        shifted = table.double()[toks[b]] * 2.5
        for t in range(9):
            for i in range((W + 1) // 2):
                a = (p0 + t) * 10000.0 ** (-2.0 * i / W)
                shifted[t, 2 * i] += math.sin(a)
                if 2 * i + 1 < W:
                    shifted[t, 2 * i + 1] += math.cos(a)
        if p0 == 0:                                                             # the oracle's own embedding counts from 0
            assert (oracle.embed(toks[b], table.double(), 2.5) - shifted).abs().max() < 1e-12
        assert (got[b].double() - shifted).abs().max() < 2e-4               # float angles at positions in the hundreds


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("rows,C,groups,shared,gate_first", [(7, 48, 4, True, False), (5, 96, 3, False, True), (70, 40, 1, False, True), (3, 66, 2, True, True),
                                                             (3, 2048, 1, False, True), (5, 4096, 2, True, False), (2, 1030, 1, False, True)])
def test_grouped_gated_norm(device, rows, C, groups, shared, gate_first):
    g = torch.Generator().manual_seed(rows)
    x, big = torch.randn(rows, C, generator=g), torch.randn(rows, C + 10, generator=g)
    gate = big[:, 5:5 + C]                                                  # a strided view, as the mixers pass it
    w = torch.randn(C // groups if shared else C, generator=g)
    out = torch.zeros(rows, C + 6)
    got = seqmix.group_rms_norm_gated(x.to(device), big.to(device)[:, 5:5 + C], w.to(device), groups, 1e-5, gate_first,
                                      out.to(device)[:, 3:3 + C], 0.6).cpu()
    xd, gd = x.double(), oracle.silu(gate.double())
    y = xd * gd if gate_first else xd
    y = oracle.rms(y.view(rows, groups, -1), 1e-5).reshape(rows, C) * (w.double().repeat(groups) if shared else w.double())
    y = (y if gate_first else y * gd) * 0.6
    assert (got.double() - y).abs().max() < 1e-5


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("taps,bias,C", [(1, False, 44), (2, True, 44), (4, True, 44), (6, False, 44), (3, True, 45), (9, False, 44)])
def test_short_conv_with_silu_prompt_then_tokens(device, taps, bias, C):
    g = torch.Generator().manual_seed(taps)
    S = 13
    x, w = torch.randn(1, S, C, generator=g), torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    want = oracle.silu(oracle.causal_conv(x[0].double(), w.double(), None if b is None else b.double()))
    state = torch.zeros(3, taps - 1, C, device=device)
    dv = lambda t: None if t is None else t.to(device)
    one = lambda v: torch.tensor([v], dtype=torch.int32, device=device)
    got = [seqmix.short_conv(x[:, :5].to(device), dv(w), dv(b), state, one(2), one(5), True, False, torch.float32, True)]
    for t in range(5, S):
        got.append(seqmix.short_conv(x[:, t:t + 1].to(device), dv(w), dv(b), state, one(2), one(1), False, False, torch.float32, True))
    assert (torch.cat(got, 1)[0].cpu().double() - want).abs().max() < 1e-5


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("N,E,top,n_real,act", [(7, 12, 4, 8, "softmax"), (40, 5, 5, 5, "softmax"), (3, 70, 9, 64, "softmax"), (9, 33, 2, 30, "sigmoid"), (1, 200, 8, 199, "softmax")])
def test_router_scores_choice_and_identity_share(device, N, E, top, n_real, act):
    g = torch.Generator().manual_seed(E)
    logits, corr = torch.randn(N, E, generator=g) * 2, torch.randn(E, generator=g) * 0.2
    w, idx, ident = seqmix.route_topk(logits.to(device), corr.to(device), top, n_real, act, 1.5)
    sc = torch.softmax(logits.double(), -1) if act == "softmax" else torch.sigmoid(logits.double())
    want = torch.topk(sc + corr.double(), top).indices
    assert torch.equal(idx.cpu(), want)                                        # descending by corrected score
    ws = sc.gather(1, want)
    assert (w.cpu().double() - torch.where(want < n_real, ws * 1.5, 0 * ws)).abs().max() < 1e-6
    assert (ident.cpu().double() - torch.where(want >= n_real, ws, 0 * ws).sum(1)).abs().max() < 1e-6


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("N,O,I", [(1, 9, 48), (5, 3, 130), (16, 40, 64), (40, 7, 33)])
def test_float_result_products(device, N, O, I):
    g = torch.Generator().manual_seed(N * O)
    big, w = torch.randn(N, I + 6, generator=g), torch.randn(O, I, generator=g)
    got = seqmix.linear_f32(big.to(device)[:, 3:3 + I], w.to(device)).cpu()
    assert got.dtype == torch.float32 and (got.double() - big[:, 3:3 + I].double() @ w.double().T).abs().max() < 1e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("M,F,I", [(5, 7, 50), (40, 64, 48), (3, 33, 131)])
def test_gated_expert_pieces(device, M, F, I):
    """``silu(gate) * up`` as an elementwise kernel and inside the expert-streaming product, vector and element-wise layouts; rows
    that name no expert give zeros."""
    g = torch.Generator().manual_seed(M * F)
    gu = torch.randn(M, 2 * F, generator=g)
    want = oracle.silu(gu[:, :F].double()) * gu[:, F:].double()
    assert (seqmix.silu_mul(gu.to(device)).cpu().double() - want).abs().max() < 1e-6
    E = 4
    w, x = torch.randn(E, 2 * F, I, generator=g) / math.sqrt(I), torch.randn(M, I, generator=g)
    sel = torch.randint(-1, E + 1, (M,), generator=g).to(torch.int32)
    got = seqmix.indexed_gemv(w.to(device), sel.to(device), x.to(device), "silu_glu").cpu().double()
    for m in range(M):
        if 0 <= int(sel[m]) < E:
            y = w[int(sel[m])].double() @ x[m].double()
            assert (got[m] - oracle.silu(y[:F]) * y[F:]).abs().max() < 1e-5
        else:
            assert (got[m] == 0).all()


def _ffn(f, width, device, seed, dtype=torch.float32):
    cfg = make_cfg([par(mlp=f)], width=width)
    w = random_checkpoint(cfg, seed)
    r = f["router"]
    m = RoutedFFN(width, f["expert"]["ff"], r["experts"], r["top"], router_act="softmax", gated=True, identity_experts=r.get("identity", 0),
                  choice_bias=True, dtype=dtype, device=torch.device(device))
    P = oracle.sub(w, "l0.mlp.")
    with torch.no_grad():
        m.up.copy_(torch.stack([torch.cat([P[f"e{e}.gate"], P[f"e{e}.up"]]) for e in range(r["experts"])]))
        m.down.copy_(torch.stack([P[f"e{e}.down"] for e in range(r["experts"])]))
        m.router.linear_router.weight.copy_(P["router"])
        m.correction.copy_(P["correction"])
    return m, P


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("rows,experts,identity,top", [(5, 5, 2, 3), (70, 5, 2, 3), (40, 4, 0, 1), (9, 2, 4, 6), (33, 6, 1, 2)])
def test_routed_ffn_choice_bias_and_identity_experts(device, rows, experts, identity, top):
    f = moe(experts, identity, top)
    m, P = _ffn(f, 48, device, rows)
    h = torch.randn(rows, 48, generator=torch.Generator().manual_seed(rows))
    # the correction must change some choices, or the test would not see it being left out or entering the weights
    s = torch.softmax(h.double() @ P["router"].double().T, -1)
    assert (torch.topk(s, top).indices.sort().values != torch.topk(s + P["correction"].double(), top).indices.sort().values).any() or top == experts + identity
    want = oracle.moe(h.double(), {k: v.double() for k, v in P.items()}, f)
    assert (m(h.to(device)).cpu().double() - want).abs().max() < 1e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,G,D,V,window,softcap", [(4, 2, 24, 40, 7, 20.0), (3, 3, 48, 96, 33, 0.0), (6, 1, 8, 130, 1, 5.0), (2, 2, 72, 16, 64, 30.0), (2, 1, 40, 300, 9, 10.0)])
def test_window_attention_prompt_and_ring(device, H, G, D, V, window, softcap):
    """The attention ops alone: a batch of prompts of unequal lengths, then single tokens against the rings, with a gate and scale."""
    g = torch.Generator().manual_seed(H * D)
    B, S, extra = 3, 45, 40
    lens = [45, 1, 20]
    T = S + extra
    q, k, v, gate = (torch.randn(B, T, n, d, generator=g) for n, d in ((H, D), (G, D), (G, V), (H, 1)))
    qw, kw = torch.randn(D, generator=g) * 0.3 + 1, torch.randn(D, generator=g) * 0.3 + 1
    scale, ring = 1.3 / math.sqrt(D), min(window, 4096)
    # expected, per sequence over its real tokens
    want = []
    for b in range(B):
        n = lens[b] + extra
        qq = oracle.rms(q[b, :n].double(), 1e-5) * qw.double()
        kk = oracle.rms(k[b, :n].double(), 1e-5) * kw.double()
        o = torch.zeros(n, H, V, dtype=torch.float64)
        for i in range(n):
            lo = max(0, i - window + 1)
            for h in range(H):
                sc = (kk[lo:i + 1, h // (H // G)] @ qq[i, h]) * scale
                sc = softcap * torch.tanh(sc / softcap) if softcap > 0 else sc
                o[i, h] = (torch.softmax(sc, 0)[:, None] * v[b, lo:i + 1, h // (H // G)].double()).sum(0) * torch.sigmoid(gate[b, i, h, 0].double()) * 0.8
        want.append(o.reshape(n, H * V))
    kc, vc = torch.zeros(5, ring, G, D, device=device), torch.zeros(5, ring, G, V, device=device)
    kc.fill_(float("nan")), vc.fill_(float("nan"))                          # whatever a slot held must never be read
    slots = [4, 0, 2]
    dv = lambda t: t.to(device)
    ctx = ctx_for(lens, slots, [0, 0, 0], True, device)
    qs, ks, vs = dv(q[:, :S].clone()), dv(k[:, :S].clone()), dv(v[:, :S].clone())
    seqmix.window_qk_prepare(qs, ks, vs, dv(qw), dv(kw), 1e-5, ctx.pos0, ctx.lens, ctx.slots, kc, vc)
    out = torch.zeros(B * S, H * V + 8, device=device)
    seqmix.window_attention_prompt(qs, ks, vs, dv(gate[:, :S, :, 0]), ctx.lens, window, scale, softcap, out[:, 4:4 + H * V], 0.8)
    got = out[:, 4:4 + H * V].view(B, S, -1).cpu()
    for b in range(B):
        assert (got[b, :lens[b]].double() - want[b][:lens[b]]).abs().max() < 2e-5
        assert (got[b, lens[b]:] == 0).all()
    for t in range(extra):
        pos = [n + t for n in lens]
        ctx = ctx_for([1, 1, 1], slots, pos, False, device)
        idx = torch.tensor(pos)
        pick = lambda a: dv(torch.stack([a[b, pos[b]] for b in range(B)])[:, None].clone())
        q1, k1, v1, g1 = pick(q), pick(k), pick(v), pick(gate)[..., 0]
        seqmix.window_qk_prepare(q1, k1, v1, dv(qw), dv(kw), 1e-5, ctx.pos0, ctx.lens, ctx.slots, kc, vc)
        o1 = torch.zeros(B, H * V, device=device)
        seqmix.window_attention_token(q1, kc, vc, g1, ctx.slots, ctx.pos0, ctx.lens, window, scale, softcap, o1, 0.8)
        for b in range(B):
            assert (o1[b].cpu().double() - want[b][pos[b]]).abs().max() < 2e-5, (b, t)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,G,D,V,window,ring", [(4, 2, 32, 48, 300, 300), (6, 1, 16, 24, 700, 700), (2, 2, 40, 8, 1000, 260)])
def test_single_token_attention_over_long_rings(device, H, G, D, V, window, ring):
    """Rings long enough for the kernel to split them into stretches: positions before the ring is full, at its last row, just
    after the first wrap and far later, against an explicit sum over the positions the ring rows hold."""
    g = torch.Generator().manual_seed(ring)
    pos = [5, ring - 1, ring, 3 * ring + 17] if ring == window else [5, ring - 1, 100, 259]
    B = len(pos)
    kc, vc = torch.randn(B + 1, ring, G, D, generator=g), torch.randn(B + 1, ring, G, V, generator=g)
    q, gate = torch.randn(B, 1, H, D, generator=g), torch.randn(B, 1, H, generator=g)
    slots, scale, cap = [3, 0, 4, 1], 1.7 / math.sqrt(D), 12.0
    out = torch.zeros(B, H * V, device=device)
    ctx = ctx_for([1] * B, slots, pos, False, device)
    seqmix.window_attention_token(q.to(device), kc.to(device), vc.to(device), gate.to(device), ctx.slots, ctx.pos0, ctx.lens, window, scale, cap, out, 1.0)
    for b in range(B):
        js = [j for j in range(max(0, pos[b] - window + 1), pos[b] + 1)]
        for h in range(H):
            kk = torch.stack([kc[slots[b], j % ring, h // (H // G)] for j in js]).double()
            vv = torch.stack([vc[slots[b], j % ring, h // (H // G)] for j in js]).double()
            sc = cap * torch.tanh((kk @ q[b, 0, h].double()) * scale / cap)
            want = (torch.softmax(sc, 0)[:, None] * vv).sum(0) * torch.sigmoid(gate[b, 0, h].double())
            assert (out[b, h * V:(h + 1) * V].cpu().double() - want).abs().max() < 2e-5, (b, h)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,G,D,V", [(4, 2, 20, 12), (2, 2, 64, 64), (3, 1, 9, 70), (1, 1, 130, 33)])
def test_gated_delta_scan_rows_of_many_lengths_and_a_carried_state(device, H, G, D, V):
    g = torch.Generator().manual_seed(D)
    B, S = 3, 21
    lens = [21, 0, 9]
    q, k, v = torch.randn(B, S, G, D, generator=g), torch.randn(B, S, G, D, generator=g), torch.randn(B, S, H, V, generator=g)
    ba = torch.randn(B, S, 2 * H, generator=g) * 2
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5 - 1, torch.randn(H, generator=g)
    s0 = torch.randn(6, H, D, V, generator=g)
    state = s0.clone().to(device)
    dv = lambda t: t.to(device)
    ctx = ctx_for(lens, [5, 1, 3], [0, 0, 0], False, device)
    got = seqmix.gated_delta_scan(dv(q), dv(k), dv(v), dv(ba)[..., :H], dv(ba)[..., H:], dv(a_log), dv(dt_bias), state, ctx.slots, ctx.lens, False).cpu()
    for b, slot in enumerate([5, 1, 3]):
        M = s0[slot].double()
        for t in range(lens[b]):
            for h in range(H):
                qq, kk = q[b, t, h // (H // G)].double(), k[b, t, h // (H // G)].double()
                qq, kk = qq / torch.sqrt((qq * qq).sum() + 1e-6) * D ** -0.5, kk / torch.sqrt((kk * kk).sum() + 1e-6)
                dec = torch.exp(-torch.exp(a_log[h].double()) * oracle.softplus(ba[b, t, H + h].double() + dt_bias[h].double()))
                M[h] = dec * M[h]
                u = torch.sigmoid(ba[b, t, h].double()) * (v[b, t, h].double() - M[h].T @ kk)
                M[h] = M[h] + torch.outer(kk, u)
                assert (got[b, t, h].double() - M[h].T @ qq).abs().max() < 1e-4
        assert (got[b, lens[b]:] == 0).all()
        assert (state[slot].cpu().double() - M).abs().max() < 1e-4
    assert torch.equal(state[[0, 2, 4]].cpu(), s0[[0, 2, 4]])                 # other slots are not touched


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,G,N,V", [(4, 2, 10, 12), (2, 1, 64, 64), (3, 3, 33, 70), (8, 2, 130, 8)])
def test_ssd_scan_rows_of_many_lengths_and_a_carried_state(device, H, G, N, V):
    g = torch.Generator().manual_seed(N)
    B, S = 3, 19
    lens = [19, 4, 0]
    x, bm, cm = torch.randn(B, S, H, V, generator=g), torch.randn(B, S, G, N, generator=g), torch.randn(B, S, G, N, generator=g)
    dt = torch.randn(B, S, H, generator=g)
    a_log, dt_bias, dskip = torch.randn(H, generator=g) * 0.5 - 0.5, torch.randn(H, generator=g), torch.randn(H, generator=g)
    s0 = torch.randn(4, H, N, V, generator=g)
    state = s0.clone().to(device)
    dv = lambda t: t.to(device)
    ctx = ctx_for(lens, [2, 0, 3], [0, 0, 0], False, device)
    got = seqmix.ssd_scan(dv(x), dv(bm), dv(cm), dv(dt), dv(a_log), dv(dt_bias), dv(dskip), state, ctx.slots, ctx.lens, False).cpu()
    for b, slot in enumerate([2, 0, 3]):
        M = s0[slot].double()
        for t in range(lens[b]):
            for h in range(H):
                step = oracle.softplus(dt[b, t, h].double() + dt_bias[h].double())
                M[h] = torch.exp(-torch.exp(a_log[h].double()) * step) * M[h] + step * torch.outer(bm[b, t, h // (H // G)].double(), x[b, t, h].double())
                y = M[h].T @ cm[b, t, h // (H // G)].double() + dskip[h].double() * x[b, t, h].double()
                assert (got[b, t, h].double() - y).abs().max() < 1e-4
        assert (state[slot].cpu().double() - M).abs().max() < 1e-4
    assert torch.equal(state[1].cpu(), s0[1])


SINGLE = {
    "parallel": [par()],
    "parallel_equal_heads_no_cap": [par(left_spec(heads=3, kv_heads=3, softcap=0.0, window=4), right_spec(heads=3, kv_heads=3, conv=2), ls=1.0, rs=1.0)],
    "parallel_one_kv_head_wide": [par(left_spec(heads=4, kv_heads=1, dim=72, vdim=136, window=50), right_spec(heads=2, kv_heads=1, dim=72, vdim=40, conv=4))],
    "ssm": [ssm()],
    "ssm_one_group_one_tap": [ssm(heads=3, vdim=20, state=7, groups=1, norm_groups=3, conv=1)],
    "ssm_group_per_head": [ssm(heads=2, vdim=8, state=40, groups=2, norm_groups=1, conv=2)],
    "moe_after_ssm": [ssm(mlp=moe())],
    "moe_all_chosen": [par(mlp=moe(experts=2, identity=1, top=3))],
}


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_single_layer_models(device, name):
    """One layer of each kind: the whole prompt at once, and one token followed by token-by-token decoding, against the oracle."""
    cfg = make_cfg(SINGLE[name], width=48 if "wide" not in name else 64)
    w = random_checkpoint(cfg, seed=len(name))
    toks = tokens_for(cfg, 26, 5)
    want, _ = oracle.forward(cfg, w, toks)
    model = build(cfg, w, device)
    close(run_alone(model, toks, len(toks)), want, TOL32)
    close(run_alone(model, toks, 1), want, TOL32)


# ------------------------------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def mixed():
    cfg = make_cfg(MIXED)
    w = random_checkpoint(cfg, seed=11)
    toks = tokens_for(cfg, 48, 7)
    want, stream = oracle.forward(cfg, w, toks)
    return cfg, w, toks, want, stream


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [48, 1, 2, 6, 31])
def test_prompt_then_decode_matches_oracle(device, mixed, prompt):
    cfg, w, toks, want, _ = mixed
    close(run_alone(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_residual_stream_after_every_layer(device, mixed):
    cfg, w, toks, _, stream = mixed
    model = build(cfg, w, device)
    seen = {}
    model.forward_step(torch.tensor([toks], device=device), [len(toks)], [model.states.alloc()], [0], True, tap=lambda i, x: seen.__setitem__(i, x[0].cpu().clone()))
    for i in range(len(MIXED)):
        close(seen[i], stream[i], TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_unequal_batch_against_each_alone_and_reused_slots(device, mixed):
    cfg, w, toks, _, _ = mixed
    model = build(cfg, w, device)
    reqs = [tokens_for(cfg, n, 20 + n) for n in (1 + 6, 7 + 6, 23 + 6, 2 + 6)]
    prompts, steps = [1, 7, 23, 2], [0, 6, 3, 6]                      # row 0 ends with its prompt, row 2 leaves early
    mgr = model.states
    warm = [mgr.alloc() for _ in range(3)]                            # dirty a few slots first, then give them back
    model.forward_step(torch.randint(0, 50, (3, 9), device=device), [9, 9, 9], warm, [0, 0, 0], True)
    for s in warm:
        mgr.free(s)
    slots = [mgr.alloc() for _ in reqs]
    assert set(warm) <= set(slots)
    S = max(prompts)
    ids = torch.zeros(len(reqs), S, dtype=torch.long)
    for b, (r, p) in enumerate(zip(reqs, prompts)):
        ids[b, :p] = torch.tensor(r[:p])
    x = model.forward_step(ids.to(device), prompts, slots, [0] * len(reqs), True)
    got = [[model.logits(x[b, :p]).cpu()] for b, p in enumerate(prompts)]
    live = [b for b in range(len(reqs)) if steps[b] > 0]
    mgr.free(slots[0])
    for k in range(max(steps)):
        live = [b for b in live if k < steps[b]]
        step_ids = torch.tensor([[reqs[b][prompts[b] + k]] for b in live], device=device)
        x = model.forward_step(step_ids, [1] * len(live), [slots[b] for b in live], [prompts[b] + k for b in live], False)
        lg = model.logits(x[:, 0]).cpu()
        for j, b in enumerate(live):
            got[b].append(lg[j:j + 1])
    for b, r in enumerate(reqs):
        n = prompts[b] + steps[b]
        want, _ = oracle.forward(cfg, w, r[:n])
        close(torch.cat(got[b]), want, TOL32)
    fresh = build(cfg, w, device)
    close(torch.cat(got[2]), run_alone(fresh, reqs[2][:26], 23), 1e-5)      # the batch changes nothing beyond rounding


# ------------------------------------------------------------------------------------------------- edges, far keys, long decoding
def _needle_model(layers, vocab=40, width=48, seed=3):
    """Token 0 is the needle: its embedding is large and unlike the others, so wherever a layer can still see it the logits move."""
    cfg = make_cfg(layers, vocab=vocab, width=width)
    w = random_checkpoint(cfg, seed=seed)
    w["embed"][0] = (w["embed"][0] * 12).to(torch.bfloat16).float()
    return cfg, w


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [40, 12, 1])
def test_window_edges_with_a_needle(device, prompt):
    """The needle sits at position 9 of a model whose only path to the past is attention with window 6 (the recurrent branch has
    weight 0): positions 9..14 see it, 15 on do not.  Checked in a prompt, and with the edge passing over decoded tokens."""
    window, at = 6, 9
    cfg, w = _needle_model([par(left_spec(window=window), rs=0.0), par(left_spec(heads=2, kv_heads=1, dim=8, vdim=16, window=window), rs=0.0)])
    toks = [1 + t % 7 for t in range(40)]
    plain = list(toks)
    toks[at] = 0
    want, _ = oracle.forward(cfg, w, toks)
    base, _ = oracle.forward(cfg, w, plain)
    moved = (want - base).abs().amax(-1)
    reach = at + 2 * (window - 1)                                      # two layers: the needle's trace travels two windows
    assert (moved[at:at + window] > 1e-2).all() and (moved[reach + 1:] < 1e-9).all() and (moved[:at] < 1e-9).all()
    assert moved[reach] > 1e-6
    close(run_alone(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("layer", ["delta", "ssm"])
def test_far_key_through_a_recurrent_state(device, layer):
    """A needle 250 tokens back is still in the state: slow decays, a long prompt, then decoding; a lost or restarted state shows."""
    if layer == "delta":
        cfg, w = _needle_model([par(left_spec(window=3), right_spec(heads=2, kv_heads=1, dim=16, vdim=16), ls=0.3)], seed=5)
        w["l0.mix.right.A_log"] = torch.full_like(w["l0.mix.right.A_log"], -7.0)       # decay close to 1: long memory
        w["l0.mix.right.b"] = w["l0.mix.right.b"] * 0 - 0.0                             # beta = 1/2 everywhere
    else:
        cfg, w = _needle_model([ssm(heads=2, vdim=16, state=16, groups=1, norm_groups=1)], seed=5)
        w["l0.mix.A_log"] = torch.full_like(w["l0.mix.A_log"], -7.0)
    toks = [1 + (t * 5) % 11 for t in range(280)]
    plain = list(toks)
    toks[4] = 0
    want, _ = oracle.forward(cfg, w, toks)
    base, _ = oracle.forward(cfg, w, plain)
    assert (want[-1] - base[-1]).abs().max() > 1e-3                         # the far token still matters at the end
    model = build(cfg, w, device)
    close(run_alone(model, toks, 250), want, TOL32)
    close(run_alone(model, toks, 280), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_from_one_token(device):
    cfg = make_cfg([par(left_spec(window=16), mlp=moe(top=2)), ssm(mlp=None), par(left_spec(window=40, heads=2, kv_heads=2), mlp=moe(experts=3, identity=1, top=1))])
    w = random_checkpoint(cfg, seed=21)
    toks = tokens_for(cfg, 130, 9)
    want, _ = oracle.forward(cfg, w, toks)
    close(run_alone(build(cfg, w, device), toks, 1), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_window_larger_than_the_cache_limit(device):
    """``max_seq_len`` below the window: the ring is only as long as sequences can get."""
    cfg = make_cfg([par(left_spec(window=500))])
    w = random_checkpoint(cfg, seed=2)
    toks = tokens_for(cfg, 30, 3)
    want, _ = oracle.forward(cfg, w, toks)
    model = build(cfg, w, device, max_seq_len=30)
    assert model.states.layer(0)["left.k"].shape[1] == 30
    close(run_alone(model, toks, 11), want, TOL32)


def test_continuing_step_carries_one_token(mixed):
    cfg, w, toks, _, _ = mixed
    model = build(cfg, w, "cpu")
    s = model.states.alloc()
    model.forward_step(torch.tensor([toks[:4]]), [4], [s], [0], True)
    with pytest.raises(ValueError):
        model.forward_step(torch.tensor([toks[4:7]]), [3], [s], [4], False)


# ---------------------------------------------------------------------------------------------- generation, registry, command lines
def _oracle_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        lg, _ = oracle.forward(cfg, w, toks)
        toks.append(int(lg[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_serving_entry_points(device, mixed):
    cfg, w, _, _, _ = mixed
    prompts = [tokens_for(cfg, 9, 31), tokens_for(cfg, 4, 32)]
    want = [_oracle_greedy(cfg, w, p, 5) for p in prompts]
    model = build(cfg, w, device, batch_size=2)
    model.on_device_sampling = True
    ids = torch.zeros(2, 9, dtype=torch.long)
    mask = torch.zeros(2, 9, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    out = model.generate(ids.to(device), 5, prompt_lens=mask.sum(1).to(device))
    assert out.cpu().tolist() == want
    out = HuggingFaceGenerationAdapter(model, pad_token_id=0).generate(ids.to(device), attention_mask=mask.to(device), max_new_tokens=5)
    assert out[:, 9:].cpu().tolist() == want


def _save_model_dir(path, cfg, w):
    from neuronx_distributed_b200.utils.safetensors_utils import save_state_dict_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_state_dict_safetensors({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))


def _trace(cfg):
    a, b, c = tokens_for(cfg, 14, 41), tokens_for(cfg, 5, 42), tokens_for(cfg, 9, 43)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": [0, 9]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []}]
    for k in range(4):
        ent = [{"id": "a", "tokens": [a[10 + k]], "want": [0]}]
        if k < 2:
            ent.append({"id": "b", "tokens": [b[3 + k]], "want": [] if k == 0 else [0]})
        steps.append({"step": k + 1, "entries": ent, "end": (["b"] if k == 1 else []) + (["a"] if k == 3 else [])})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": c, "want": [8]}], "end": ["c"]})
    rows = {0: [("a", 0), ("a", 9), ("b", 2)], 1: [("a", 10)], 2: [("a", 11), ("b", 4)], 3: [("a", 12)], 4: [("a", 13)], 5: [("c", 8)]}
    return {"a": a, "b": b, "c": c}, steps, rows


@pytest.mark.parametrize("device", DEVICES)
def test_registry_checkpoint_reader_and_trace_replay(device, mixed, tmp_path):
    import numpy as np

    cfg, w, _, _, _ = mixed
    _save_model_dir(str(tmp_path / "m"), cfg, w)
    model = registry.load_for_serving(str(tmp_path / "m"), dtype=torch.float32, device=torch.device(device), max_seq_len=64, on_device_sampling=False)
    assert isinstance(model, PiniraxForInference)
    reqs, steps, rows = _trace(cfg)
    out = tmp_path / "o"
    os.makedirs(out)
    import io

    log = io.StringIO()
    TraceReplayer(model, str(out)).run([json.dumps(s) for s in steps], log)
    assert log.getvalue().split() == [x for s in steps for x in ("done", str(s["step"]))]
    assert model.states.in_use == 0
    for n, want_rows in rows.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(want_rows), cfg["vocab"]).copy())
        for j, (rid, pos) in enumerate(want_rows):
            want, _ = oracle.forward(cfg, w, reqs[rid][:pos + 1])
            close(got[j:j + 1], want[-1:], TOL32)


def test_trace_runner_command_line(mixed, tmp_path):
    import numpy as np

    cfg, w, _, _, _ = mixed
    _save_model_dir(str(tmp_path / "m"), cfg, w)
    reqs, steps, rows = _trace(cfg)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--out", str(tmp_path / "o"),
                        "--max-tokens", "40"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got = np.fromfile(tmp_path / "o" / "5.f32", dtype="<f4")
    want, _ = oracle.forward(cfg, w, reqs["c"])
    close(torch.from_numpy(got.copy())[None], want[8:9], TOL32)


def test_generate_command_line(mixed, tmp_path):
    cfg, w, _, _, _ = mixed
    _save_model_dir(str(tmp_path / "m"), cfg, w)
    prompts = [tokens_for(cfg, 6, 51), tokens_for(cfg, 3, 52)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    args = [os.path.join(ROOT, "bin", "generate"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--max-new-tokens", "4"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(t) for t in line.split(",")] for line in r.stdout.strip().splitlines()[-2:]]
    assert got == [_oracle_greedy(cfg, w, p, 4) for p in prompts]


# ---------------------------------------------------------------------------------------------------------------- bfloat16 (GPU)
@pytest.mark.gpu
def test_bfloat16_serving_close_to_the_oracle():
    cfg = make_cfg([par(left_spec(window=9), mlp=None), ssm(mlp=None), par(mlp=None)], width=64)
    w = random_checkpoint(cfg, seed=13)
    toks = tokens_for(cfg, 40, 3)
    want, _ = oracle.forward(cfg, w, toks)
    model = build(cfg, w, "cuda", dtype=torch.bfloat16)
    close(run_alone(model, toks, 25), want, 5e-2)
    close(run_alone(model, toks, 40), want, 5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [6, 300])
def test_bfloat16_routed_ffn_rows_with_a_clear_choice(rows):
    """bfloat16 rows whose routing is not a close call (router logits spread out): streaming and per-expert paths against the oracle."""
    f = moe(experts=6, identity=2, top=2, ff=64)
    m, P = _ffn(f, 128, "cuda", 3, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(rows)
    h = torch.randn(rows, 128, generator=g).to(torch.bfloat16)
    s = torch.softmax(h.double() @ P["router"].double().T, -1) + P["correction"].double()
    top3 = torch.topk(s, 3).values
    keep = (top3[:, 1] - top3[:, 2]) > 0.02                                # the second and third choices are well apart
    h = h[keep]
    want = oracle.moe(h.double(), {k: v.double() for k, v in P.items()}, f)
    got = m(h.cuda()).cpu().double()
    assert ((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("H,G,D,V", [(4, 2, 16, 32), (6, 2, 48, 96), (2, 1, 128, 128), (3, 3, 64, 16), (2, 2, 256, 256)])
@pytest.mark.parametrize("window,softcap", [(1, 30.0), (7, 0.0), (64, 5.0), (100, 50.0), (1000, 20.0)])
def test_bfloat16_prompt_attention_in_one_kernel(H, G, D, V, window, softcap):
    """The fused tensor-core prompt kernel (bfloat16, sizes in whole 16s) against the float statement of the same op on the same
    rounded inputs: unequal lengths, tiles cut by the window and by the end of a sequence, strided operands, gate and scale."""
    g = torch.Generator().manual_seed(D + window)
    B, S = 3, 200
    lens = torch.tensor([200, 77, 1], dtype=torch.int32)
    P = H * D + G * (D + V) + 8
    p = (torch.randn(B, S, P, generator=g) * 1.5).to(torch.bfloat16)
    q, k, v = p[..., :H * D].unflatten(-1, (H, D)), p[..., H * D:H * D + G * D].unflatten(-1, (G, D)), p[..., H * D + G * D:H * D + G * (D + V)].unflatten(-1, (G, V))
    gate = p[..., -8:-8 + H]
    scale = 2.0 / math.sqrt(D)
    want = torch.zeros(B * S, H * V)
    seqmix.window_attention_prompt(q.float(), k.float(), v.float(), gate.float(), lens, window, scale, softcap, want, 0.8)
    pc = p.cuda()
    qc, kc, vc = pc[..., :H * D].unflatten(-1, (H, D)), pc[..., H * D:H * D + G * D].unflatten(-1, (G, D)), pc[..., H * D + G * D:H * D + G * (D + V)].unflatten(-1, (G, V))
    out = torch.full((B * S, H * V + 16), 7.0, dtype=torch.bfloat16, device="cuda")
    seqmix.window_attention_prompt(qc, kc, vc, pc[..., -8:-8 + H], lens.cuda(), window, scale, softcap, out[:, 8:8 + H * V], 0.8)
    got = out[:, 8:8 + H * V].float().cpu()
    assert (out[:, :8] == 7).all() and (out[:, 8 + H * V:] == 7).all()
    assert (got - want).abs().max() < 0.03 * max(1.0, want.abs().max().item())
    assert ((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 1e-2
    for b in range(B):
        assert (got.view(B, S, -1)[b, lens[b]:] == 0).all()
