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
