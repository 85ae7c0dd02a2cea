"""Naguzen: a decoder-only language model whose layers mix three kinds of sequence mixer — latent sliding-window attention
(``modules/attention/latent_attention.py``), gated linear attention (``modules/recurrent/gla.py``) and a real-gated LRU block
(``modules/recurrent/rglru.py``) — with dense (xIELU) or routed (sigmoid top-k, erf-GELU experts + shared expert) feed-forwards.

Block shape: the norm sits on the sublayer's OUTPUT, ``x += norm1(mixer(cv1(x)))`` then ``x += norm2(ff(cv2(x)))`` with
``cv(h) = h + conv(h)`` a short causal convolution per channel and ``norm`` an RMS norm with a single gain.  The residual stream
``x`` is float; the sublayers compute in the model dtype.  Every layer therefore carries state per sequence: two convolution
histories, plus a ring cache (attention) or a float recurrent state (+ a third history in the LRU block).  ``config.json`` lists the
layers in order (``type``, ``mixer`` sizes, ``mlp``), so any order and any sizes load without code changes.

Serving follows ``LlamaForInference``: ``context_encoding`` (right-padded prompts) / ``token_generation`` (one token per row) /
``generate``; state lives in a ``SequenceStateManager`` (slots handed to requests and reused)."""
from __future__ import annotations

import dataclasses
import json
import math
import os
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from ..inference.slot_serving import SlotServingModel
from ..inference.state_cache import SequenceStateManager, StepContext  # noqa: F401  (StepContext is re-exported)
from ..modules.attention.latent_attention import LatentWindowAttention
from ..modules.moe.routed_ffn import RoutedFFN
from ..modules.recurrent import GatedLinearAttention, RealGatedLRUBlock
from ..modules.rms_norm import ScalarRMSNorm
from ..modules.short_conv import ShortConv
from ..ops import act, seqmix
from ..utils.sampling import Sampler


@dataclasses.dataclass
class NaguzenConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]                    # [{"type", "mixer": {...}, "mlp": {...} | None}, ...] as in config.json
    norm_eps: float = 1e-6
    canon_taps: int = 4
    dtype: torch.dtype = torch.bfloat16
    device: Any = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any], **overrides) -> "NaguzenConfig":
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=list(d["layers"]), norm_eps=float(d["norm"]["eps"]),
                   canon_taps=int(d["canon"]["taps"]), **overrides)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "NaguzenConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f), **overrides)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


class DenseFFN(nn.Module):
    """``W_down xielu(W_up h)``; the activation's two raw parameters are turned into its positive coefficients at load time."""

    def __init__(self, width: int, ff: int, dtype, device=None):
        super().__init__()
        self.up = nn.Parameter(torch.zeros(ff, width, dtype=dtype, device=device), requires_grad=False)
        self.down = nn.Parameter(torch.zeros(width, ff, dtype=dtype, device=device), requires_grad=False)
        self.alpha_pos, self.alpha_neg = 1.0, 1.0

    def set_activation(self, raw: torch.Tensor) -> None:
        sp = F.softplus(raw.float())
        self.alpha_pos, self.alpha_neg = float(sp[0]), float(0.5 + sp[1])

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return F.linear(act.xielu(F.linear(h, self.up), self.alpha_pos, self.alpha_neg), self.down)


def _build_mixer(cfg: NaguzenConfig, spec: Dict[str, Any], max_seq_len: int) -> nn.Module:
    m, kind = spec["mixer"], spec["type"]
    if kind == "latent_attention":
        return LatentWindowAttention(cfg.width, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"],
                                     window=int(m["mask"]["size"]), scale=float(m["scale"]), rot_base=float(m["rot"]["base"]),
                                     rot_dims=int(m["rot"]["dims"]), eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device,
                                     max_seq_len=max_seq_len)
    if kind == "gla":
        return GatedLinearAttention(cfg.width, m["heads"], m["dim"], m["vdim"], decay_rank=int(m["decay_rank"]), tau=float(m["tau"]),
                                    eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device)
    if kind == "rglru":
        return RealGatedLRUBlock(cfg.width, m["width"], m["blocks"], int(m["conv"]), dtype=cfg.dtype, device=cfg.device)
    raise ValueError(f"unknown mixer type {kind!r}")


def _build_ffn(cfg: NaguzenConfig, f: Optional[Dict[str, Any]]) -> Optional[nn.Module]:
    if not f:
        return None
    if f["kind"] == "dense":
        return DenseFFN(cfg.width, int(f["ff"]), cfg.dtype, cfg.device)
    if f["kind"] == "moe":
        r = f["router"]
        return RoutedFFN(cfg.width, int(f["expert"]["ff"]), int(r["experts"]), int(r["top"]), weight_scale=float(r.get("scale", 1.0)),
                         shared_ff=int((f.get("shared") or {}).get("ff", 0)), dtype=cfg.dtype, device=cfg.device)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


class NaguzenLayer(nn.Module):
    def __init__(self, cfg: NaguzenConfig, spec: Dict[str, Any], max_seq_len: int):
        super().__init__()
        self.kind, self.dtype = spec["type"], cfg.dtype
        self.canon1 = ShortConv(cfg.width, cfg.canon_taps, residual=True, device=cfg.device)
        self.mixer = _build_mixer(cfg, spec, max_seq_len)
        self.norm1 = ScalarRMSNorm(cfg.norm_eps, cfg.device)
        self.mlp = _build_ffn(cfg, spec.get("mlp"))
        if self.mlp is not None:
            self.canon2 = ShortConv(cfg.width, cfg.canon_taps, residual=True, device=cfg.device)
            self.norm2 = ScalarRMSNorm(cfg.norm_eps, cfg.device)

    def state_spec(self):
        spec = {"canon1": self.canon1.state_spec(torch.float32)}
        spec.update(self.mixer.state_spec())
        if self.mlp is not None:
            spec["canon2"] = self.canon2.state_spec(torch.float32)
        return spec

    def forward(self, x: torch.Tensor, ctx: StepContext, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        """``x [B,S,width]`` float residual stream, updated in place."""
        B, S, W = x.shape
        h = self.canon1(x, st["canon1"], ctx, self.dtype)
        self.norm1.add_to(x, self.mixer(h, ctx, st))
        if self.mlp is not None:
            h = self.canon2(x, st["canon2"], ctx, self.dtype)
            self.norm2.add_to(x, self.mlp(h.view(B * S, W)))
        return x


class NaguzenForCausalLM(nn.Module):
    def __init__(self, cfg: NaguzenConfig, max_seq_len: int = 1 << 30):
        super().__init__()
        self.cfg = self.config = cfg
        self.embed = nn.Parameter(torch.zeros(cfg.vocab, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)
        self.layers = nn.ModuleList([NaguzenLayer(cfg, spec, max_seq_len) for spec in cfg.layers])
        self.norm = ScalarRMSNorm(cfg.norm_eps, cfg.device)
        self.head = nn.Parameter(torch.zeros(cfg.vocab, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)

    def state_specs(self):
        return [layer.state_spec() for layer in self.layers]

    def body(self, input_ids: torch.Tensor, ctx: StepContext, states: SequenceStateManager, tap=None) -> torch.Tensor:
        x = F.embedding(input_ids, self.embed).float()
        for i, layer in enumerate(self.layers):
            x = layer(x, ctx, states.layer(i))
            if tap is not None:
                tap(i, x)
        return x

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        """Residual rows ``[n, width]`` float → float logits ``[n, vocab]``."""
        return F.linear(self.norm(rows, out_dtype=self.cfg.dtype), self.head).float()


# --------------------------------------------------------------------------------------------------------------- checkpoint names
def convert_state_dict(cfg: NaguzenConfig, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (``embed``, ``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``;
    linear weights ``[out, in]``) → this module's parameters: projections that read the same input are stacked, per-head matrices
    get a head axis, experts are stacked, gate matrices are transposed, and everything the kernels read as float is float."""
    out: Dict[str, torch.Tensor] = {"embed": sd["embed"], "head": sd["head"], "norm.weight": sd["final.norm"]}
    for i, spec in enumerate(cfg.layers):
        p, o, m = f"l{i}.", f"layers.{i}.", spec["mixer"]
        out[o + "norm1.weight"], out[o + "canon1.weight"] = sd[p + "norm1"], sd[p + "canon1"]
        x = lambda n: sd[p + "mix." + n]
        if spec["type"] == "latent_attention":
            H = m["heads"]
            for a, b in (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"), ("o", "o")):
                out[o + "mixer." + a] = x(b)
            out[o + "mixer.uk"] = x("uk").view(H, m["dim"], m["kv_rank"])
            out[o + "mixer.uv"] = x("uv").view(H, m["vdim"], m["kv_rank"])
        elif spec["type"] == "gla":
            out[o + "mixer.in_proj"] = torch.cat([x("q"), x("k"), x("v"), x("g"), x("a1")], 0)
            out[o + "mixer.a2"], out[o + "mixer.a2_bias"] = x("a2"), x("a2.b")
            out[o + "mixer.norm"], out[o + "mixer.o"] = x("norm"), x("o")
        elif spec["type"] == "rglru":
            out[o + "mixer.in_proj"] = torch.cat([x("y"), x("x")], 0)
            out[o + "mixer.in_bias"] = torch.cat([x("y.b"), x("x.b")], 0)
            out[o + "mixer.conv.weight"], out[o + "mixer.conv.bias"] = x("conv"), x("conv.b")
            out[o + "mixer.gate_r"], out[o + "mixer.gate_i"] = x("ra").transpose(1, 2).contiguous(), x("ri").transpose(1, 2).contiguous()
            out[o + "mixer.gate_r_bias"], out[o + "mixer.gate_i_bias"] = x("ra.b").reshape(-1), x("ri.b").reshape(-1)
            out[o + "mixer.lam_softplus"] = F.softplus(x("lam").float())
            out[o + "mixer.o"] = x("o")
        f = spec.get("mlp")
        if not f:
            continue
        out[o + "norm2.weight"], out[o + "canon2.weight"] = sd[p + "norm2"], sd[p + "canon2"]
        y = lambda n: sd[p + "mlp." + n]
        if f["kind"] == "dense":
            out[o + "mlp.up"], out[o + "mlp.down"], out[o + "mlp.act"] = y("up"), y("down"), y("act")
        else:
            E = f["router"]["experts"]
            out[o + "mlp.up"] = torch.stack([y(f"e{e}.up") for e in range(E)])
            out[o + "mlp.down"] = torch.stack([y(f"e{e}.down") for e in range(E)])
            out[o + "mlp.router.linear_router.weight"] = y("router")
            if f.get("shared"):
                out[o + "mlp.shared_up"], out[o + "mlp.shared_down"] = y("shared.up"), y("shared.down")
    return out


def complete_config(d: Dict[str, Any], shapes: Dict[str, Sequence[int]]) -> Dict[str, Any]:
    """Sizes that ``config.json`` leaves to the tensors' shapes (the decay projection's rank of a gla layer)."""
    d = json.loads(json.dumps(d))
    for i, spec in enumerate(d["layers"]):
        if spec["type"] == "gla" and "decay_rank" not in spec["mixer"]:
            spec["mixer"]["decay_rank"] = int(shapes[f"l{i}.mix.a1"][0])
        if spec["type"] == "rglru":
            spec["mixer"]["conv"] = int(shapes[f"l{i}.mix.conv"][1])
    return d


def load_naguzen_weights(model: NaguzenForCausalLM, sd: Dict[str, torch.Tensor]) -> None:
    conv = convert_state_dict(model.cfg, sd)
    acts = {k: conv.pop(k) for k in [k for k in conv if k.endswith("mlp.act")]}
    params = dict(model.named_parameters())
    missing = sorted(set(params) - set(conv))
    extra = sorted(set(conv) - set(params))
    if missing or extra:
        raise KeyError(f"checkpoint does not fit the model: missing {missing[:6]}, unexpected {extra[:6]}")
    with torch.no_grad():
        for k, v in conv.items():
            if tuple(params[k].shape) != tuple(v.shape):
                raise ValueError(f"{k}: checkpoint shape {tuple(v.shape)} != {tuple(params[k].shape)}")
            params[k].copy_(v.to(params[k].dtype))
        for k, v in acts.items():
            model.get_submodule(k[: -len(".act")]).set_activation(v)


# ------------------------------------------------------------------------------------------------------------------------ serving
class NaguzenForInference(SlotServingModel):
    def __init__(self, cfg: NaguzenConfig, batch_size: int = 1, max_seq_len: int = 2048, on_device_sampling: bool = True,
                 sampler: Optional[Sampler] = None):
        super().__init__(cfg, NaguzenForCausalLM(cfg, max_seq_len=max_seq_len), batch_size=batch_size, max_seq_len=max_seq_len,
                         on_device_sampling=on_device_sampling, sampler=sampler)

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "NaguzenForInference":
        from ..utils.safetensors_utils import load_state_dict_safetensors

        sd = load_state_dict_safetensors(os.path.join(path, "model.safetensors"))
        with open(os.path.join(path, "config.json")) as f:
            d = complete_config(json.load(f), {k: tuple(v.shape) for k, v in sd.items()})
        model = cls(NaguzenConfig.from_dict(d, dtype=dtype, device=device), **kw)
        load_naguzen_weights(model.lm, sd)
        return model.eval()

    def load_checkpoint_tensors(self, sd) -> None:
        load_naguzen_weights(self.lm, sd)
