"""Grouped-query softmax attention over a sliding window, without positional rotation: biased q/k/v projections, an RMS norm per
head on queries and keys (one weight vector each, shared by the heads), scores ``q.k * scale`` optionally capped as
``softcap * tanh(score / softcap)``, and one sigmoid output gate per head read from the layer's input.  Position i sees
``i - window < j <= i``, so each sequence keeps a ring of ``window`` key and value rows (``csrc/seqmix/window_attention.cu``).

q, k, v and the gate logits are one stacked projection of the input; the norm, the ring store and the attention read their
parts of it in place through strides.  ``mix`` writes the gated heads (times a caller's scale) into a caller's buffer so that a
layer that sums several mixers can run ONE output projection over all of them; ``forward`` is the stand-alone layer."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class GatedWindowAttention(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, window: int, scale: float, softcap: float = 0.0,
                 eps: float = 1e-6, qk_norm: bool = True, head_gate: bool = True, dtype: torch.dtype = torch.bfloat16, device=None,
                 max_seq_len: int = 1 << 30):
        super().__init__()
        assert heads % kv_heads == 0, "query heads must divide into the key/value heads"
        self.heads, self.kv_heads, self.dim, self.vdim = heads, kv_heads, dim, vdim
        self.window, self.scale, self.softcap, self.eps, self.dtype = int(window), float(scale), float(softcap), eps, dtype
        self.ring = max(1, min(self.window, max_seq_len))
        self.head_gate = head_gate
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.ones(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.n_q, self.n_k, self.n_v = heads * dim, kv_heads * dim, kv_heads * vdim
        rows = self.stacked_rows(heads, kv_heads, dim, vdim, head_gate)
        self.in_proj, self.in_bias = mk(rows, width), mk(rows)                       # rows: q | k | v | gate | zero padding
        self.q_norm, self.k_norm = (f32(dim), f32(dim)) if qk_norm else (None, None)
        self.o = mk(width, heads * vdim)

    @staticmethod
    def stacked_rows(heads: int, kv_heads: int, dim: int, vdim: int, head_gate: bool = True) -> int:
        """Rows of the stacked projection: q | k | v | gate, padded to a whole 8 so that token rows stay 16-byte aligned in bfloat16
        (the fused prompt kernel reads q, k and v in place)."""
        n = heads * dim + kv_heads * (dim + vdim) + (heads if head_gate else 0)
        return -(-n // 8) * 8

    @property
    def out_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"k": ((self.ring, self.kv_heads, self.dim), self.dtype), "v": ((self.ring, self.kv_heads, self.vdim), self.dtype)}

    def mix(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor], out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        """``h [B,S,width]`` → the gated heads times ``out_scale`` in ``out [B*S, heads*vdim]`` (a view with any row stride)."""
        B, S, _ = h.shape
        if not ctx.fresh and S != 1:
            raise ValueError("window attention continues a sequence one token at a time")
        H, G, D, V = self.heads, self.kv_heads, self.dim, self.vdim
        p = F.linear(h, self.in_proj, self.in_bias)
        a, b, c = self.n_q, self.n_q + self.n_k, self.n_q + self.n_k + self.n_v
        q, k, v = p[..., :a].unflatten(-1, (H, D)), p[..., a:b].unflatten(-1, (G, D)), p[..., b:c].unflatten(-1, (G, V))
        gate = p[..., c:c + H] if self.head_gate else None
        seqmix.window_qk_prepare(q, k, v, self.q_norm, self.k_norm, self.eps, ctx.pos0, ctx.lens, ctx.slots, st["k"], st["v"])
        if ctx.fresh:
            return seqmix.window_attention_prompt(q, k, v, gate, ctx.lens, self.window, self.scale, self.softcap, out, out_scale)
        return seqmix.window_attention_token(q, st["k"], st["v"], gate, ctx.slots, ctx.pos0, ctx.lens, self.window, self.scale,
                                             self.softcap, out, out_scale)

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        heads = torch.empty(B * S, self.out_features, dtype=h.dtype, device=h.device)
        return F.linear(self.mix(h, ctx, st, heads), self.o).view(B, S, -1)
