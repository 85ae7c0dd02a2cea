"""Pinirax: a decoder-only language model whose layers put a pair of sequence mixers side by side — grouped-query sliding-window
attention with capped scores and a gate per head (``modules/attention/window_attention.py``) next to a gated delta rule
(``modules/recurrent/delta_rule.py``), summed with fixed weights (``modules/parallel_mixers.py``) — or a selective state space
mixer (``modules/recurrent/ssd.py``), each followed by a routed feed-forward of gated experts whose softmax router has a
choice-only correction and identity experts (``modules/moe/routed_ffn.py``).

Block shape: a norm on both sides of every sublayer, ``x += norm1b(mixer(norm1(x)))`` then ``x += norm2b(ff(norm2(x)))``, all RMS
norms whose stored weight is the gain's offset from one.  The embedding is scaled and gets interleaved sinusoids of the position
added (no rotation anywhere).  The residual stream ``x`` is float; the sublayers compute in the model dtype.  ``config.json``
lists the layers in order (``type``, ``mixer`` sizes, ``mlp`` or null), so any order and any sizes load without code changes.

Serving is the slot-based wrapper shared with the other stateful families (``inference/slot_serving.py``)."""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from ..inference.slot_serving import SlotServingModel
from ..inference.state_cache import SequenceStateManager, StepContext
from ..modules.attention.window_attention import GatedWindowAttention
from ..modules.moe.routed_ffn import RoutedFFN
from ..modules.parallel_mixers import ParallelMixers
from ..modules.recurrent import GatedDeltaRule, SelectiveStateSpace
from ..modules.rms_norm import OffsetRMSNorm
from ..ops import seqmix
from ..utils.sampling import Sampler

SINUSOID_BASE = 10000.0


@dataclasses.dataclass
class PiniraxConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]                    # [{"type", "mixer": {...}, "mlp": {...} | None}, ...] as in config.json
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    dtype: torch.dtype = torch.bfloat16
    device: Any = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any], **overrides) -> "PiniraxConfig":
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=list(d["layers"]), norm_eps=float(d["norm"]["eps"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), **overrides)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "PiniraxConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f), **overrides)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def _build_mixer(cfg: PiniraxConfig, spec: Dict[str, Any], max_seq_len: int) -> nn.Module:
    m, kind = spec["mixer"], spec["type"]
    if kind == "parallel":
        l, r = m["left"], m["right"]
        left = GatedWindowAttention(cfg.width, int(l["heads"]), int(l["kv_heads"]), int(l["dim"]), int(l["vdim"]),
                                    window=int(l["mask"]["size"]), scale=float(l.get("scale", int(l["dim"]) ** -0.5)),
                                    softcap=float(l.get("softcap", 0.0)),
                                    eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device, max_seq_len=max_seq_len)
        right = GatedDeltaRule(cfg.width, int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"]), int(r["conv"]),
                               eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device)
        return ParallelMixers({"left": left, "right": right}, [float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))])
    if kind == "mamba2":
        return SelectiveStateSpace(cfg.width, int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["norm_groups"]),
                                   int(m["conv"]), eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device)
    raise ValueError(f"unknown mixer type {kind!r}")


def _build_ffn(cfg: PiniraxConfig, f: Optional[Dict[str, Any]]) -> Optional[nn.Module]:
    if not f:
        return None
    if f["kind"] == "moe":
        r = f["router"]
        return RoutedFFN(cfg.width, int(f["expert"]["ff"]), int(r["experts"]), int(r["top"]), router_act="softmax", gated=True,
                         identity_experts=int(r.get("identity", 0)), choice_bias=True, dtype=cfg.dtype, device=cfg.device)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


class PiniraxLayer(nn.Module):
    def __init__(self, cfg: PiniraxConfig, spec: Dict[str, Any], max_seq_len: int):
        super().__init__()
        self.kind, self.dtype = spec["type"], cfg.dtype
        self.norm1, self.norm1b = OffsetRMSNorm(cfg.width, cfg.norm_eps, cfg.device), OffsetRMSNorm(cfg.width, cfg.norm_eps, cfg.device)
        self.mixer = _build_mixer(cfg, spec, max_seq_len)
        self.mlp = _build_ffn(cfg, spec.get("mlp"))
        if self.mlp is not None:
            self.norm2, self.norm2b = OffsetRMSNorm(cfg.width, cfg.norm_eps, cfg.device), OffsetRMSNorm(cfg.width, cfg.norm_eps, cfg.device)

    def state_spec(self):
        return self.mixer.state_spec()

    def forward(self, x: torch.Tensor, ctx: StepContext, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        """``x [B,S,width]`` float residual stream, updated in place."""
        B, S, W = x.shape
        self.norm1b.add_to(x, self.mixer(self.norm1(x, out_dtype=self.dtype), ctx, st))
        if self.mlp is not None:
            self.norm2b.add_to(x, self.mlp(self.norm2(x, out_dtype=self.dtype).view(B * S, W)))
        return x


class PiniraxForCausalLM(nn.Module):
    def __init__(self, cfg: PiniraxConfig, max_seq_len: int = 1 << 30):
        super().__init__()
        self.cfg = self.config = cfg
        self.embed = nn.Parameter(torch.zeros(cfg.vocab, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)
        self.register_buffer("inv_freq", seqmix.sinusoid_inv_freq(cfg.width, SINUSOID_BASE, cfg.device), persistent=False)
        self.layers = nn.ModuleList([PiniraxLayer(cfg, spec, max_seq_len) for spec in cfg.layers])
        self.norm = OffsetRMSNorm(cfg.width, cfg.norm_eps, cfg.device)
        self.head = nn.Parameter(torch.zeros(cfg.vocab, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)

    def state_specs(self):
        return [layer.state_spec() for layer in self.layers]

    def body(self, input_ids: torch.Tensor, ctx: StepContext, states: SequenceStateManager, tap=None) -> torch.Tensor:
        x = seqmix.embed_sinusoid(input_ids, self.embed, self.cfg.embedding_scale, self.inv_freq, ctx.pos0)
        for i, layer in enumerate(self.layers):
            x = layer(x, ctx, states.layer(i))
            if tap is not None:
                tap(i, x)
        return x

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        """Residual rows ``[n, width]`` float → float logits ``[n, vocab]``."""
        return F.linear(self.norm(rows, out_dtype=self.cfg.dtype), self.head).float()


# --------------------------------------------------------------------------------------------------------------- checkpoint names
def convert_state_dict(cfg: PiniraxConfig, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``;
    linear weights ``[out, in]``) → this module's parameters: projections that read the same input are stacked (missing biases are
    zeros), experts are stacked with the gate rows over the up rows, the convolutions of one mixer are stacked, and everything the
    kernels read as float is float.  Norm offsets are returned under ``*.offset`` keys and turned into gains by the loader."""
    out: Dict[str, torch.Tensor] = {"embed": sd["embed"], "head": sd["head"], "norm.offset": sd["final.norm"]}
    for i, spec in enumerate(cfg.layers):
        p, o, m = f"l{i}.", f"layers.{i}.", spec["mixer"]
        out[o + "norm1.offset"], out[o + "norm1b.offset"] = sd[p + "norm1"], sd[p + "norm1b"]
        x = lambda n: sd[p + "mix." + n]
        if spec["type"] == "parallel":
            a, b = o + "mixer.branches.left.", o + "mixer.branches.right."
            H = int(m["left"]["heads"])
            stack = torch.cat([x("left.q"), x("left.k"), x("left.v"), x("left.g")], 0)
            pad = GatedWindowAttention.stacked_rows(H, int(m["left"]["kv_heads"]), int(m["left"]["dim"]), int(m["left"]["vdim"])) - stack.shape[0]
            out[a + "in_proj"] = torch.cat([stack, stack.new_zeros(pad, stack.shape[1])], 0)
            out[a + "in_bias"] = torch.cat([x("left.q.b"), x("left.k.b"), x("left.v.b"), torch.zeros(H + pad, dtype=x("left.q.b").dtype)], 0)
            out[a + "q_norm"], out[a + "k_norm"], out[a + "o"] = x("left.q.norm"), x("left.k.norm"), x("left.o")
            out[b + "in_proj"] = torch.cat([x("right.q"), x("right.k"), x("right.v"), x("right.g")], 0)
            out[b + "ba_proj"] = torch.cat([x("right.b"), x("right.a")], 0)
            out[b + "conv.weight"] = torch.cat([x("right.q.conv"), x("right.k.conv"), x("right.v.conv")], 0)
            out[b + "a_log"], out[b + "dt_bias"] = x("right.A_log"), x("right.dt_bias")
            out[b + "norm"], out[b + "o"] = x("right.norm"), x("right.o")
        elif spec["type"] == "mamba2":
            a = o + "mixer."
            nh = int(m["heads"])
            out[a + "in_proj"], out[a + "dt_proj"] = x("in")[:-nh], x("in")[-nh:]
            out[a + "conv.weight"], out[a + "conv.bias"] = x("conv"), x("conv.b")
            out[a + "a_log"], out[a + "dt_bias"], out[a + "d_skip"] = x("A_log"), x("dt_bias"), x("D")
            out[a + "norm"], out[a + "o"] = x("norm"), x("o")
        f = spec.get("mlp")
        if not f:
            continue
        out[o + "norm2.offset"], out[o + "norm2b.offset"] = sd[p + "norm2"], sd[p + "norm2b"]
        y = lambda n: sd[p + "mlp." + n]
        E = int(f["router"]["experts"])
        out[o + "mlp.up"] = torch.stack([torch.cat([y(f"e{e}.gate"), y(f"e{e}.up")], 0) for e in range(E)])
        out[o + "mlp.down"] = torch.stack([y(f"e{e}.down") for e in range(E)])
        out[o + "mlp.router.linear_router.weight"], out[o + "mlp.correction"] = y("router"), y("correction")
    return out


def complete_config(d: Dict[str, Any], shapes: Dict[str, Sequence[int]]) -> Dict[str, Any]:
    """Sizes that a ``config.json`` may leave to the tensors' shapes (the taps of the short convolutions)."""
    d = json.loads(json.dumps(d))
    for i, spec in enumerate(d["layers"]):
        if spec["type"] == "parallel" and "conv" not in spec["mixer"]["right"]:
            spec["mixer"]["right"]["conv"] = int(shapes[f"l{i}.mix.right.q.conv"][1])
        if spec["type"] == "mamba2" and "conv" not in spec["mixer"]:
            spec["mixer"]["conv"] = int(shapes[f"l{i}.mix.conv"][1])
    return d


def load_pinirax_weights(model: PiniraxForCausalLM, sd: Dict[str, torch.Tensor]) -> None:
    conv = convert_state_dict(model.cfg, sd)
    offsets = {k[: -len(".offset")]: conv.pop(k) for k in [k for k in conv if k.endswith(".offset")]}
    params = dict(model.named_parameters())
    have = set(conv) | {k + ".weight" for k in offsets}
    missing, extra = sorted(set(params) - have), sorted(have - set(params))
    if missing or extra:
        raise KeyError(f"checkpoint does not fit the model: missing {missing[:6]}, unexpected {extra[:6]}")
    with torch.no_grad():
        for k, v in conv.items():
            if tuple(params[k].shape) != tuple(v.shape):
                raise ValueError(f"{k}: checkpoint shape {tuple(v.shape)} != {tuple(params[k].shape)}")
            params[k].copy_(v.to(params[k].dtype))
        for k, v in offsets.items():
            model.get_submodule(k).set_offset(v)


# ------------------------------------------------------------------------------------------------------------------------ serving
class PiniraxForInference(SlotServingModel):
    def __init__(self, cfg: PiniraxConfig, batch_size: int = 1, max_seq_len: int = 2048, on_device_sampling: bool = True,
                 sampler: Optional[Sampler] = None):
        super().__init__(cfg, PiniraxForCausalLM(cfg, max_seq_len=max_seq_len), batch_size=batch_size, max_seq_len=max_seq_len,
                         on_device_sampling=on_device_sampling, sampler=sampler)

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "PiniraxForInference":
        from ..utils.safetensors_utils import load_state_dict_safetensors

        sd = load_state_dict_safetensors(os.path.join(path, "model.safetensors"))
        with open(os.path.join(path, "config.json")) as f:
            d = complete_config(json.load(f), {k: tuple(v.shape) for k, v in sd.items()})
        model = cls(PiniraxConfig.from_dict(d, dtype=dtype, device=device), **kw)
        load_pinirax_weights(model.lm, sd)
        return model.eval()

    def load_checkpoint_tensors(self, sd) -> None:
        load_pinirax_weights(self.lm, sd)
