"""Naguzen serving path against the plain oracle (tests/naguzen_oracle.py): every mechanism alone, whole prompts, prompt + token by
token decoding, unequal batches, reused slots, window edges, far keys, other sizes, greedy generation through the serving entry
points, the registry / checkpoint reader and the trace runner.  Configurations and weights are made here (random, seeded)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import naguzen_oracle as oracle  # noqa: E402

from neuronx_distributed_b200.inference.hf_adapter import HuggingFaceGenerationAdapter  # noqa: E402
from neuronx_distributed_b200.inference.state_cache import SequenceStateManager  # noqa: E402
from neuronx_distributed_b200.inference.trace_replay import TraceReplayer  # noqa: E402
from neuronx_distributed_b200.models import registry  # noqa: E402
from neuronx_distributed_b200.models.naguzen import (NaguzenConfig, NaguzenForInference, StepContext, complete_config,  # noqa: E402
                                                     load_naguzen_weights)
from neuronx_distributed_b200.modules.moe.routed_ffn import RoutedFFN  # noqa: E402
from neuronx_distributed_b200.ops import seqmix  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


# ------------------------------------------------------------------------------------------------------------------ model making
def attn_spec(heads=3, dim=24, rot=8, vdim=40, kv_rank=48, q_rank=56, window=7, base=1000.0, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot}, "scale": 1.0 / math.sqrt(dim + rot)}}


def gla_spec(heads=3, dim=20, vdim=12, tau=7.0, mlp=None):
    return {"type": "gla", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def lru_spec(width=96, blocks=3, conv=3, mlp=None):
    return {"type": "rglru", "mlp": mlp, "mixer": {"width": width, "blocks": blocks, "conv": conv}}


DENSE = {"kind": "dense", "ff": 72}


def moe(experts=6, top=3, scale=1.7, ff=24, shared=40):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def make_cfg(layers, vocab=50, width=48, taps=3, eps=1e-5):
    return {"architecture": "Naguzen", "vocab": vocab, "width": width, "canon": {"taps": taps}, "norm": {"eps": eps}, "layers": layers}


def random_checkpoint(cfg, seed=0, decay_rank=5):
    g = torch.Generator().manual_seed(seed)
    bf = lambda t: t.to(torch.bfloat16).float()
    lin = lambda o, i, s=1.0: bf(torch.randn(o, i, generator=g) * s / math.sqrt(i))
    vec = lambda n, s=1.0, m=0.0: bf(torch.randn(n, generator=g) * s + m)
    W, w = cfg["width"], {}
    w["embed"], w["head"], w["final.norm"] = bf(torch.randn(cfg["vocab"], W, generator=g)), lin(cfg["vocab"], W), bf(torch.tensor(1.3))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"], w[p + "canon1"] = bf(torch.tensor(0.9)), bf(torch.randn(W, cfg["canon"]["taps"], generator=g) * 0.3)
        if L["type"] == "latent_attention":
            H, D, R, V, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w.update({p + "mix.dq": lin(Q, W), p + "mix.dq.norm": vec(Q, 0.2, 1.0), p + "mix.uq": lin(H * (D + R), Q, 2.0),
                      p + "mix.dkv": lin(C + R, W, 2.0), p + "mix.dkv.norm": vec(C, 0.2, 1.0), p + "mix.uk": lin(H * D, C, 2.0),
                      p + "mix.uv": lin(H * V, C), p + "mix.o": lin(W, H * V)})
        elif L["type"] == "gla":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": lin(H * D, W), p + "mix.k": lin(H * D, W), p + "mix.v": lin(H * V, W), p + "mix.g": lin(H * V, W),
                      p + "mix.o": lin(W, H * V), p + "mix.norm": vec(V, 0.2, 1.0), p + "mix.a1": lin(decay_rank, W),
                      p + "mix.a2": lin(H * D, decay_rank, 2.0), p + "mix.a2.b": vec(H * D, 1.0, 2.0)})
        else:
            RW, nb, taps = m["width"], m["blocks"], m["conv"]
            w.update({p + "mix.y": lin(RW, W), p + "mix.y.b": vec(RW, 0.1), p + "mix.x": lin(RW, W), p + "mix.x.b": vec(RW, 0.1),
                      p + "mix.conv": bf(torch.randn(RW, taps, generator=g) * 0.5), p + "mix.conv.b": vec(RW, 0.1),
                      p + "mix.ra": bf(torch.randn(nb, RW // nb, RW // nb, generator=g) / math.sqrt(RW // nb)), p + "mix.ra.b": bf(torch.randn(nb, RW // nb, generator=g)),
                      p + "mix.ri": bf(torch.randn(nb, RW // nb, RW // nb, generator=g) / math.sqrt(RW // nb)), p + "mix.ri.b": bf(torch.randn(nb, RW // nb, generator=g)),
                      p + "mix.lam": vec(RW, 1.0, -2.0), p + "mix.o": lin(W, RW)})
        f = L.get("mlp")
        if not f:
            continue
        w[p + "norm2"], w[p + "canon2"] = bf(torch.tensor(1.1)), bf(torch.randn(W, cfg["canon"]["taps"], generator=g) * 0.3)
        if f["kind"] == "dense":
            w.update({p + "mlp.up": lin(f["ff"], W), p + "mlp.down": lin(W, f["ff"]), p + "mlp.act": bf(torch.tensor([0.3, -0.4]))})
        else:
            for e in range(f["router"]["experts"]):
                w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = lin(f["expert"]["ff"], W), lin(W, f["expert"]["ff"])
            w[p + "mlp.router"] = lin(f["router"]["experts"], W, 3.0)
            if f.get("shared"):
                w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = lin(f["shared"]["ff"], W), lin(W, f["shared"]["ff"])
    return w


def build(cfg, weights, device, dtype=torch.float32, max_seq_len=4096, batch_size=1):
    full = complete_config(cfg, {k: tuple(v.shape) for k, v in weights.items()})
    m = NaguzenForInference(NaguzenConfig.from_dict(full, dtype=dtype, device=torch.device(device)), batch_size=batch_size,
                            max_seq_len=max_seq_len, on_device_sampling=False)
    load_naguzen_weights(m.lm, weights)
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
    """Mean-free difference relative to the spread of the expected logits, per position."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    ref = (want - want.mean(-1, keepdim=True)).double().pow(2).mean().sqrt()
    err = (d.pow(2).mean(-1).sqrt() / ref).max().item()
    assert err < tol, f"relative error {err:.3e} >= {tol}"


MIXED = [gla_spec(mlp=moe()), attn_spec(mlp=DENSE), lru_spec(mlp=moe(experts=4, top=1, shared=0)), attn_spec(window=5, heads=2, mlp=None),
         gla_spec(heads=1, dim=8, vdim=24, tau=2.0, mlp=DENSE)]
TOL32 = 2e-4


# ------------------------------------------------------------------------------------------------------------ single mechanisms
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("taps,residual,bias", [(1, True, False), (3, True, False), (4, False, True), (6, False, False)])
def test_short_conv_prompt_then_tokens(device, taps, residual, bias):
    g = torch.Generator().manual_seed(taps)
    B, S, C, extra = 3, 9, 40, 5
    lens = [9, 1, 4]
    x = torch.randn(B, S + extra, C, generator=g)
    w, b = torch.randn(C, taps, generator=g), (torch.randn(C, generator=g) if bias else None)
    state = torch.full((5, taps - 1, C), 7.0)                                   # stale contents must be ignored by a fresh call
    slots = torch.tensor([4, 0, 2], dtype=torch.int32)
    dv = lambda t: None if t is None else t.to(device)
    st = state.to(device)
    out = seqmix.short_conv(dv(x[:, :S].contiguous()), dv(w), dv(b), st, dv(slots), dv(torch.tensor(lens, dtype=torch.int32)), True,
                            residual, torch.float32).cpu()
    got = [[out[i, t] for t in range(lens[i])] for i in range(B)]
    for k in range(extra):                                                      # continue every row by single tokens
        step = torch.stack([x[i, lens[i] + k] for i in range(B)])[:, None]
        o = seqmix.short_conv(dv(step.contiguous()), dv(w), dv(b), st, dv(slots), dv(torch.ones(B, dtype=torch.int32)), False, residual,
                              torch.float32).cpu()
        for i in range(B):
            got[i].append(o[i, 0])
    for i in range(B):
        seq = x[i, : lens[i] + extra].double()
        want = oracle.short_conv(seq, w.double()) + (b.double() if bias else 0) + (seq if residual else 0)
        assert torch.allclose(torch.stack(got[i]).double(), want, atol=1e-5), (i, taps)
    assert (out[1, 1:] == 0).all() and (out[2, 4:] == 0).all()                  # padding rows are zeros


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("rows,C", [(11, 70), (3, 520), (5, 515), (1300, 72), (1200, 516)])
def test_norms_and_activations(device, rows, C):
    """Few and many rows, narrow and wide, in whole fours and not: every launch shape of the norm kernels."""
    g = torch.Generator().manual_seed(1)
    x, gate, res = torch.randn(rows, C, generator=g) * 3, torch.randn(rows, C, generator=g), torch.randn(rows, C, generator=g)
    w, one = torch.rand(C, generator=g) + 0.5, torch.tensor([0.37])
    eps = 1e-3
    dv = lambda t: t.to(device)
    want = oracle.rms(x.double(), eps)
    assert torch.allclose(seqmix.rms_norm(dv(x), dv(w), eps).cpu().double(), want * w, atol=1e-5)
    assert torch.allclose(seqmix.rms_norm(dv(x), dv(one), eps).cpu().double(), want * 0.37, atol=1e-5)
    gated = seqmix.rms_norm(dv(x), dv(w), eps, gate=dv(gate)).cpu().double()
    assert torch.allclose(gated, want * w * (gate * torch.sigmoid(gate)).double(), atol=1e-5)
    wide = torch.randn(rows, C + 20, generator=g)                               # a norm over the first columns of wider rows
    assert torch.allclose(seqmix.rms_norm(dv(wide)[:, :C], dv(w), eps).cpu().double(), oracle.rms(wide[:, :C].double(), eps) * w, atol=1e-5)
    r = dv(res.clone())
    seqmix.add_rms_norm_(r, dv(x), dv(one), eps)
    assert torch.allclose(r.cpu().double(), res.double() + want * 0.37, atol=1e-5)
    z = torch.cat([torch.randn(500, generator=g) * 3, torch.tensor([0.0, -30.0, 1e-4, -1e-4])])
    act = torch.tensor([0.3, -0.4])
    sp = torch.nn.functional.softplus(act)
    assert torch.allclose(seqmix.xielu(dv(z), float(sp[0]), float(0.5 + sp[1])).cpu().double(), oracle.xielu(z.double(), act.double()), atol=1e-5)
    assert torch.allclose(seqmix.gelu_erf(dv(z)).cpu().double(), oracle.gelu_erf(z.double()), atol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("rows,top,shared", [(5, 3, 40), (70, 3, 40), (40, 1, 0), (9, 2, 0)])
def test_routed_ffn(device, rows, top, shared):
    f = moe(experts=6, top=top, scale=1.7, ff=24, shared=shared)
    cfg = make_cfg([gla_spec(mlp=f)])
    w = random_checkpoint(cfg, seed=rows)
    P = oracle.sub(w, "l0.mlp.")
    m = RoutedFFN(cfg["width"], 24, 6, top, weight_scale=1.7, shared_ff=shared, dtype=torch.float32, device=device)
    with torch.no_grad():
        m.up.copy_(torch.stack([P[f"e{e}.up"] for e in range(6)]))
        m.down.copy_(torch.stack([P[f"e{e}.down"] for e in range(6)]))
        m.router.linear_router.weight.copy_(P["router"])
        if shared:
            m.shared_up.copy_(P["shared.up"]), m.shared_down.copy_(P["shared.down"])
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(3))
    want = oracle.moe_ff(h.double(), {k: v.double() for k, v in P.items()}, f)
    assert torch.allclose(m(h.to(device)).cpu().double(), want, atol=2e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("I,O", [(264, 19), (48, 7), (131, 5), (1024, 3)])
def test_expert_streaming_gemv(device, I, O):
    """Rows that each name their own matrix of a stack: inner sizes below, at and above one pass of a warp, in whole fours and not."""
    g = torch.Generator().manual_seed(I)
    w, x = torch.randn(5, O, I, generator=g), torch.randn(6, I, generator=g)
    sel = torch.tensor([4, 0, 0, 3, 1, 4])
    want = torch.einsum("moi,mi->mo", w[sel].double(), x.double())
    got = seqmix.indexed_gemv(w.to(device), sel.to(device), x.to(device), False).cpu().double()
    assert torch.allclose(got, want, atol=1e-4)
    got = seqmix.indexed_gemv(w.to(device), sel.to(device), x.to(device), True).cpu().double()
    assert torch.allclose(got, oracle.gelu_erf(want), atol=1e-4)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,window", [(11, 6), (8, 40), (17, 33)])
def test_many_heads_and_rings_of_several_chunks(device, heads, window):
    """More heads than one block of the single-token attention kernel takes, and rings longer than one of its chunks: a prompt, then
    tokens one by one until the window has passed over decoded tokens, against the oracle at every position."""
    cfg = make_cfg([attn_spec(heads=heads, dim=16, rot=8, vdim=24, kv_rank=40, q_rank=24, window=window, mlp=None)])
    w = random_checkpoint(cfg, seed=heads)
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    toks = tokens_for(cfg, window + 45, 7)
    want = oracle.forward(full, w, toks)[0]
    close(run_alone(build(cfg, w, device), toks, 5), want, TOL32)
    close(run_alone(build(cfg, w, device), toks, window + 3), want, TOL32)


def test_routed_ffn_blockwise_layout(monkeypatch):
    """The blockwise grouped path's bookkeeping (rows grouped by expert into padded blocks, and which row holds each (token, choice))
    with a stand-in for the grouped GEMM kernel: same result as the oracle, also when some experts get no rows."""
    import types

    from neuronx_distributed_b200.ops import _ext

    def grouped_gemm(x, w, b2e, block_rows, trans_b):
        assert trans_b and x.shape[0] == b2e.numel() * block_rows
        return torch.einsum("bti,boi->bto", x.view(b2e.numel(), block_rows, -1), w[b2e.long()]).reshape(x.shape[0], -1)

    fake = types.SimpleNamespace(grouped_gemm=grouped_gemm)
    monkeypatch.setattr(_ext, "_PLAN_PROXY", fake)
    for rows, experts, top in [(70, 6, 3), (33, 9, 1), (300, 4, 2)]:
        f = moe(experts=experts, top=top, scale=0.6, ff=24, shared=40)
        cfg = make_cfg([gla_spec(mlp=f)])
        P = oracle.sub(random_checkpoint(cfg, seed=rows), "l0.mlp.")
        m = RoutedFFN(cfg["width"], 24, experts, top, weight_scale=0.6, shared_ff=40, dtype=torch.float32)
        m.block_rows = 16
        m._grouped_kernels = lambda h: fake
        with torch.no_grad():
            m.up.copy_(torch.stack([P[f"e{e}.up"] for e in range(experts)]))
            m.down.copy_(torch.stack([P[f"e{e}.down"] for e in range(experts)]))
            m.router.linear_router.weight.copy_(P["router"])
            m.shared_up.copy_(P["shared.up"]), m.shared_down.copy_(P["shared.down"])
        h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(5))
        want = oracle.moe_ff(h.double(), {k: v.double() for k, v in P.items()}, f)
        assert torch.allclose(m(h).double(), want, atol=2e-5)


def _gla_plain(q, k, v, z, zb, tau, s0):
    """Token by token in float64: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t / sqrt(D), from the state s0 [H,D,V]."""
    S, H, D = q.shape
    alpha = torch.sigmoid(z.double() + zb.double()).pow(1.0 / tau).reshape(S, H, D)
    st, out = s0.double().clone(), []
    for t in range(S):
        st = alpha[t][:, :, None] * st + k[t].double()[:, :, None] * v[t].double()[:, None, :]
        out.append(torch.einsum("hdv,hd->hv", st, q[t].double()) * D ** -0.5)
    return torch.stack(out), st


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,D,V,tau,bias", [(2, 20, 12, 7.0, 2.0), (1, 40, 72, 0.5, -6.0), (3, 33, 5, 64.0, 5.0)])
def test_gla_scan_rows_of_many_lengths_and_a_carried_state(device, H, D, V, tau, bias):
    """Rows that end just before, at and just after the edges of the 64-token chunks of the long-run form, one single token, decays
    from almost 1 down to almost 0 (2^-17 per token and channel: nothing may overflow), states carried in from slots in use."""
    g = torch.Generator().manual_seed(D)
    lens = [63, 64, 65, 130, 1, 129, 200]
    B, S = len(lens), max(lens)
    p = torch.randn(B, S, H * (2 * D + V), generator=g)                      # one projection's output, as the layer makes it
    cut = lambda t: (t[..., :H * D].unflatten(-1, (H, D)), t[..., H * D:2 * H * D].unflatten(-1, (H, D)), t[..., 2 * H * D:].unflatten(-1, (H, V)))
    q, k, v = cut(p)
    z, zb = torch.randn(B, S, H * D, generator=g) * 2, torch.randn(H * D, generator=g) + bias
    slots = torch.tensor([6, 0, 3, 8, 2, 5, 1], dtype=torch.int32)
    for fresh in (True, False):
        state = torch.randn(9, H, D, V, generator=g)
        st = state.clone().to(device)
        dv = lambda t: t.to(device)
        out = seqmix.gla_scan(*cut(dv(p)), dv(z), dv(zb), tau, st, dv(slots), dv(torch.tensor(lens, dtype=torch.int32)), fresh).cpu()
        for b, n in enumerate(lens):
            s0 = torch.zeros(H, D, V) if fresh else state[slots[b]]
            want, last = _gla_plain(q[b, :n], k[b, :n], v[b, :n], z[b, :n], zb, tau, s0)
            scale = want.abs().max()
            assert (out[b, :n].double() - want).abs().max() < 2e-5 * scale, (b, n, fresh)
            assert (out[b, n:] == 0).all()
            assert (st[slots[b]].cpu().double() - last).abs().max() < 2e-5 * max(1.0, last.abs().max()), (b, n, fresh)
        assert torch.equal(st[4].cpu(), state[4]) and torch.equal(st[7].cpu(), state[7])          # slots of no row are not touched


SINGLE = {"attention": [attn_spec()], "attention_wide_window": [attn_spec(window=64, heads=1, dim=8, rot=4, vdim=8, kv_rank=100, q_rank=16)],
          "gla": [gla_spec()], "gla_one_head": [gla_spec(heads=1, dim=40, vdim=72, tau=1.0)], "rglru": [lru_spec()],
          "rglru_one_block": [lru_spec(width=40, blocks=1, conv=1)], "dense": [gla_spec(mlp=DENSE)], "moe": [lru_spec(mlp=moe())]}


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_single_layer_models(device, name):
    """One layer of each kind: the whole prompt at once, and one token followed by token-by-token decoding, against the oracle."""
    cfg = make_cfg(SINGLE[name], taps=2 if "one" in name else 3)
    w = random_checkpoint(cfg, seed=len(name))
    toks = tokens_for(cfg, 26, 5)
    want, _ = oracle.forward(complete_config(cfg, {k: v.shape for k, v in w.items()}), w, toks)
    model = build(cfg, w, device)
    close(run_alone(model, toks, len(toks)), want, TOL32)
    close(run_alone(model, toks, 1), want, TOL32)


# ------------------------------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def mixed():
    cfg = make_cfg(MIXED)
    w = random_checkpoint(cfg, seed=11)
    toks = tokens_for(cfg, 48, 7)
    want, trail = oracle.forward(complete_config(cfg, {k: v.shape for k, v in w.items()}), w, toks)
    return cfg, w, toks, want, trail


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [48, 1, 2, 6, 31])
def test_prompt_then_decode_matches_oracle(device, mixed, prompt):
    """Windows of 7 and 5 pass several times over decoded tokens; the first tokens (position < taps, < window) are covered by prompt 1, 2."""
    cfg, w, toks, want, _ = mixed
    close(run_alone(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_residual_stream_after_every_layer(device, mixed):
    cfg, w, toks, _, trail = mixed
    model = build(cfg, w, device)
    seen = []
    model.forward_step(torch.tensor([toks], device=device), [len(toks)], [model.states.alloc()], [0], True, tap=lambda i, x: seen.append(x[0].cpu().clone()))
    for i, (a, b) in enumerate(zip(seen, trail)):
        assert torch.allclose(a.double(), b, atol=2e-4, rtol=1e-4), f"layer {i}"


@pytest.mark.parametrize("device", DEVICES)
def test_unequal_batch_against_each_alone_and_reused_slots(device, mixed):
    cfg, w, toks, _, _ = mixed
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
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
        want, _ = oracle.forward(full, w, r[:n])
        close(torch.cat(got[b]), want, TOL32)
    fresh = build(cfg, w, device)
    close(torch.cat(got[2]), run_alone(fresh, reqs[2][:26], 23), 1e-5)      # the batch changes nothing beyond rounding


def test_state_manager_slots():
    mgr = SequenceStateManager([{"a": ((2, 3), torch.float32)}, {"b": ((4,), torch.bfloat16)}], num_slots=2)
    s = [mgr.alloc() for _ in range(5)]                                 # grows past the first allocation, keeping contents
    assert sorted(s) == [0, 1, 2, 3, 4] and mgr.layer(0)["a"].shape[0] >= 5 and mgr.layer(1)["b"].dtype == torch.bfloat16
    mgr.layer(0)["a"][3] = 5.0
    mgr.free(1), mgr.free(3)
    assert mgr.alloc() == 1 and mgr.alloc() == 3 and mgr.in_use == 5
    assert float(mgr.layer(0)["a"][3].sum()) == 30.0                    # a reused slot is handed out as it was left
    mgr.advance([1, 3], [4, 1])
    assert mgr.length[1] == 4 and mgr.length[3] == 1
    with pytest.raises(KeyError):
        mgr.free(7)


# ------------------------------------------------------------------------------------------------- edges, far keys, long decoding
def _needle_model(layers, vocab=40, width=48, seed=3):
    """Token 0 is the needle: its embedding is large, so wherever a layer can still see it the logits move by a lot."""
    cfg = make_cfg(layers, vocab=vocab, width=width)
    w = random_checkpoint(cfg, seed=seed)
    w["embed"][0] = (w["embed"][0] * 12).to(torch.bfloat16).float()
    return cfg, w


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [40, 12, 1])
def test_window_edges_with_a_needle(device, prompt):
    """The needle sits at position 9 of an attention-only model with window 6 (taps 1 → no other path to the past): positions 9..14
    see it, 15 on do not.  Checked in a prompt, and with the edge passing over decoded tokens."""
    window, at = 6, 9
    cfg, w = _needle_model([attn_spec(window=window, heads=2), attn_spec(window=window, heads=2, dim=8, rot=8, vdim=16, kv_rank=24, q_rank=16)])
    cfg["canon"]["taps"] = 1
    for k in [k for k in w if "canon" in k]:
        w[k] = w[k][:, :1]
    toks = [1 + t % 7 for t in range(40)]
    plain = list(toks)
    toks[at] = 0
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    want, _ = oracle.forward(full, w, toks)
    base, _ = oracle.forward(full, w, plain)
    moved = (want - base).abs().amax(-1)
    reach = at + 2 * (window - 1)                                      # two layers: the needle's trace travels two windows
    assert (moved[at:at + window] > 1e-2).all() and (moved[reach + 1:] < 1e-9).all() and (moved[:at] < 1e-9).all()
    assert moved[reach] > 1e-6
    close(run_alone(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("layer", ["gla", "rglru"])
def test_far_key_through_a_recurrent_state(device, layer):
    """A needle 300 tokens back is still in the state: slow decays, a long prompt, then decoding; a lost or restarted state shows."""
    spec = gla_spec(heads=2, dim=16, vdim=16, tau=64.0) if layer == "gla" else lru_spec(width=64, blocks=2, conv=2)
    cfg, w = _needle_model([spec], seed=5)
    if layer == "rglru":
        w["l0.mix.lam"] = torch.full_like(w["l0.mix.lam"], -7.0)            # a close to 1: long memory
    else:
        w["l0.mix.a2.b"] = torch.full_like(w["l0.mix.a2.b"], 5.0)
    toks = [1 + (t * 5) % 11 for t in range(330)]
    plain = list(toks)
    toks[4] = 0
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    want, _ = oracle.forward(full, w, toks)
    base, _ = oracle.forward(full, w, plain)
    assert (want[-1] - base[-1]).abs().max() > 1e-3                         # the far token still matters at the end
    model = build(cfg, w, device)
    close(run_alone(model, toks, 300), want, TOL32)
    close(run_alone(model, toks, 330), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_from_one_token(device):
    cfg = make_cfg([attn_spec(window=16, mlp=moe(top=2)), gla_spec(mlp=DENSE), lru_spec(mlp=None)], taps=4)
    w = random_checkpoint(cfg, seed=21)
    toks = tokens_for(cfg, 150, 9)
    want, _ = oracle.forward(complete_config(cfg, {k: v.shape for k, v in w.items()}), w, toks)
    close(run_alone(build(cfg, w, device), toks, 1), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_window_larger_than_the_cache_limit(device):
    """A window wider than the serving length: the ring is cut to the serving length and nothing wraps."""
    cfg = make_cfg([attn_spec(window=1000)])
    w = random_checkpoint(cfg, seed=2)
    toks = tokens_for(cfg, 30, 1)
    want, _ = oracle.forward(cfg, w, toks)
    model = build(cfg, w, device, max_seq_len=32)
    assert model.states.layer(0)["kv"].shape[1] == 32
    close(run_alone(model, toks, 11), want, TOL32)


# ---------------------------------------------------------------------------------------------- entry points, registry, runner
def _oracle_greedy(full, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        logits, _ = oracle.forward(full, w, seq)
        seq.append(int(logits[-1].argmax()))
    return seq[len(prompt):]


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_serving_entry_points(device, mixed):
    cfg, w, _, _, _ = mixed
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    prompts = [tokens_for(cfg, 9, 1), tokens_for(cfg, 4, 2)]
    want = [_oracle_greedy(full, w, p, 6) for p in prompts]
    model = build(cfg, w, device, batch_size=2)
    model.on_device_sampling = True
    ids = torch.zeros(2, 9, dtype=torch.long)
    mask = torch.zeros(2, 9, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    got = model.generate(ids.to(device), 6, prompt_lens=torch.tensor([9, 4], device=device))
    assert got.cpu().tolist() == want
    out = HuggingFaceGenerationAdapter(model, pad_token_id=0).generate(ids.to(device), attention_mask=mask.to(device), max_new_tokens=6)
    assert out[:, 9:].cpu().tolist() == want
    again = model.generate(ids.to(device), 6, prompt_lens=torch.tensor([9, 4], device=device))      # same slots, used again
    assert again.cpu().tolist() == want


def _save_model_dir(path, cfg, w):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    ints = {}
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))
    return path


def _trace(cfg):
    a, b, c = tokens_for(cfg, 12, 31), tokens_for(cfg, 5, 32), tokens_for(cfg, 1, 33)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [0, 8]}, {"id": "c", "tokens": c, "want": [0]},
                                     {"id": "b", "tokens": b[:3], "want": []}], "end": ["c"]}]
    for k in range(3):
        e = [{"id": "a", "tokens": [a[9 + k]], "want": [0]}]
        if k < 2:
            e.append({"id": "b", "tokens": [b[3 + k]], "want": [0] if k else []})
        steps.append({"step": k + 1, "entries": e, "end": ["b"] if k == 1 else (["a"] if k == 2 else [])})
    steps.append({"step": 4, "entries": [{"id": "d", "tokens": b, "want": [4]}], "end": ["d"]})        # a freed slot, used again
    rows = {0: [("a", 0), ("a", 8), ("c", 0)], 1: [("a", 9)], 2: [("a", 10), ("b", 4)], 3: [("a", 11)], 4: [("b", 4)]}
    return {"a": a, "b": b, "c": c}, steps, rows


@pytest.mark.parametrize("device", DEVICES)
def test_registry_checkpoint_reader_and_trace_replay(device, mixed, tmp_path):
    import numpy as np

    cfg, w, _, _, _ = mixed
    path = _save_model_dir(str(tmp_path / "model"), cfg, w)
    assert registry.family_of(cfg) == "naguzen" and "llama" in registry.families()
    model = registry.load_for_serving(path, dtype=torch.float32, device=torch.device(device), max_seq_len=64, on_device_sampling=False)
    assert isinstance(model, NaguzenForInference)
    reqs, steps, rows = _trace(cfg)
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    want = {k: oracle.forward(full, w, v)[0] for k, v in reqs.items()}
    out = tmp_path / "out"
    out.mkdir()
    rep = TraceReplayer(model, str(out))
    for s in steps:
        rep.step(s)
    assert model.states.in_use == 0
    for n, wanted in rows.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(wanted), cfg["vocab"]))
        close(got, torch.stack([want[i][p] for i, p in wanted]), TOL32)


def test_trace_runner_command_line(mixed, tmp_path):
    import numpy as np

    cfg, w, _, _, _ = mixed
    path = _save_model_dir(str(tmp_path / "model"), cfg, w)
    reqs, steps, rows = _trace(cfg)
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", str(out), "--max-tokens", "40"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600,
                       env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {n}" for n in range(5)]
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    got = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    close(got, torch.stack([oracle.forward(full, w, reqs["a"])[0][10], oracle.forward(full, w, reqs["b"])[0][4]]), TOL32)


def test_generate_command_line(mixed, tmp_path):
    """Greedy generation of an unequal batch through the command line (registry, static batch, sampler) equals the oracle's; a
    sampled run with a fixed seed repeats itself and stays inside the vocabulary."""
    cfg, w, _, _, _ = mixed
    path = _save_model_dir(str(tmp_path / "model"), cfg, w)
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    prompts = [tokens_for(cfg, 7, 41), tokens_for(cfg, 3, 42)]
    cmd = [os.path.join(ROOT, "bin", "generate"), "--model", path, "--dtype", "float32", "--max-new-tokens", "5"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    env = {**os.environ, "CUDA_VISIBLE_DEVICES": ""}
    run = lambda extra: subprocess.run(cmd + extra, capture_output=True, text=True, timeout=600, env=env)
    r = run([])
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(t) for t in line.split(",")] for line in r.stdout.strip().splitlines()[-2:]]
    assert got == [_oracle_greedy(full, w, p, 5) for p in prompts]
    a, b = run(["--do-sample", "--top-k", "8", "--temperature", "0.7", "--seed", "3"]), run(["--do-sample", "--top-k", "8", "--temperature", "0.7", "--seed", "3"])
    assert a.returncode == 0 and a.stdout == b.stdout, a.stderr[-2000:]
    assert all(0 <= int(t) < cfg["vocab"] for line in a.stdout.strip().splitlines()[-2:] for t in line.split(","))


@pytest.mark.gpu
def test_bfloat16_serving_close_to_the_oracle():
    """The serving precision: bfloat16 matrix products, float statistics / states / residual.  Prompt + decode, against float64.
    Dense feed-forwards only: a routed layer may pick another expert on a close call in bfloat16 (covered row by row below)."""
    cfg = make_cfg([gla_spec(mlp=DENSE), attn_spec(mlp=DENSE), lru_spec(mlp=DENSE), attn_spec(window=5, heads=2, mlp=None),
                    gla_spec(heads=1, dim=8, vdim=24, tau=2.0, mlp=DENSE)])
    w = random_checkpoint(cfg, seed=11)
    toks = tokens_for(cfg, 48, 7)
    want, _ = oracle.forward(complete_config(cfg, {k: v.shape for k, v in w.items()}), w, toks)
    model = build(cfg, w, "cuda", dtype=torch.bfloat16)
    close(run_alone(model, toks, 20), want, 8e-2)
    close(run_alone(model, toks, 48), want, 8e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,width,ff", [(6, 48, 24), (90, 48, 24), (90, 128, 64), (700, 64, 192)])
def test_bfloat16_routed_ffn_rows_with_a_clear_choice(rows, width, ff):
    """Few rows (streamed experts), many rows of odd sizes (an expert at a time) and many rows in whole 64s (the blockwise grouped
    GEMM, when the main extension is built) against the oracle, on the rows whose choice of experts is not a close call."""
    f = moe(experts=6, top=2, scale=1.7, ff=ff, shared=40)
    cfg = make_cfg([gla_spec(mlp=f)], width=width)
    w = random_checkpoint(cfg, seed=4)
    P = oracle.sub(w, "l0.mlp.")
    m = RoutedFFN(cfg["width"], ff, 6, 2, weight_scale=1.7, shared_ff=40, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        m.up.copy_(torch.stack([P[f"e{e}.up"] for e in range(6)])), m.down.copy_(torch.stack([P[f"e{e}.down"] for e in range(6)]))
        m.router.linear_router.weight.copy_(P["router"])
        m.shared_up.copy_(P["shared.up"]), m.shared_down.copy_(P["shared.down"])
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    want = oracle.moe_ff(h.double(), {k: v.double() for k, v in P.items()}, f)
    s = torch.sigmoid(h.double() @ P["router"].double().T).sort(-1, descending=True).values
    clear = (s[:, 1] - s[:, 2]) > 0.02
    got = m(h.cuda()).cpu().double()
    assert clear.sum() >= rows // 2
    assert torch.allclose(got[clear], want[clear], atol=3e-2, rtol=3e-2)

@pytest.mark.gpu
@pytest.mark.parametrize("heads,dim,rot,vdim,rank", [(3, 24, 8, 32, 48), (2, 64, 32, 64, 40), (1, 128, 64, 128, 96), (2, 8, 8, 16, 16)])
@pytest.mark.parametrize("window", [1, 7, 64, 100, 1000])
def test_bfloat16_prompt_attention_in_one_kernel(heads, dim, rot, vdim, rank, window):
    """The one-kernel prompt attention (scores and weights stay on chip) against the float oracle run on the same bfloat16 weights, for
    unequal prompts whose lengths sit around the kernel's 64-row tiles and windows below, at and above them; padded rows give zeros;
    the ring it leaves serves the next token."""
    from neuronx_distributed_b200.modules.attention.latent_attention import LatentWindowAttention

    spec = attn_spec(heads=heads, dim=dim, rot=rot, vdim=vdim, kv_rank=rank, q_rank=40, window=window)
    cfg = make_cfg([spec], width=64)
    w = random_checkpoint(cfg, seed=window)
    full = complete_config(cfg, {k: v.shape for k, v in w.items()})
    m = build(cfg, w, "cuda", dtype=torch.bfloat16, batch_size=4)
    att = m.lm.layers[0].mixer
    assert isinstance(att, LatentWindowAttention) and seqmix.latent_prompt_fused_ok(torch.zeros(1, device="cuda", dtype=torch.bfloat16), dim, rot, rank + rot, vdim)
    lens = [130, 64, 65, 3]
    toks = [tokens_for(cfg, n + 2, 50 + n) for n in lens]
    ids = torch.zeros(4, max(lens), dtype=torch.long)
    for b, t in enumerate(toks):
        ids[b, :lens[b]] = torch.tensor(t[:lens[b]])
    slots = [m.states.alloc() for _ in lens]
    runs = {}
    for fused in (True, False):
        att.fused_prompt = fused
        x = m.forward_step(ids.cuda(), lens, slots, [0] * 4, True)
        runs[fused] = torch.stack([m.logits(x[b, lens[b] - 1:lens[b]])[0] for b in range(4)]).cpu()
        nxt = m.forward_step(torch.tensor([[t[n]] for t, n in zip(toks, lens)]).cuda(), [1] * 4, slots, lens, False)
        runs[fused, "next"] = m.logits(nxt[:, 0]).cpu()
    want = torch.stack([oracle.forward(full, w, t[:n + 1])[0][n - 1:n + 1] for t, n in zip(toks, lens)])
    for fused in (True, False):
        close(runs[fused], want[:, 0], 4e-2)
        close(runs[fused, "next"], want[:, 1], 4e-2)
    close(runs[True], runs[False], 2e-2)
