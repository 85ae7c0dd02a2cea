"""Gated linear attention: per head a matrix state ``S [dim, vdim]`` with a data-dependent decay per KEY channel,
``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``, ``alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau)`` (a low-rank decay
projection).  Each head's output is RMS-normed over ``vdim`` (one weight vector shared by the heads), gated by ``silu(W_g h)`` and
projected out.  q, k, v, g and the decay's down-projection are one fused matrix product."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class GatedLinearAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay_rank: int, tau: float, eps: float,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        self.heads, self.dim, self.vdim, self.decay_rank, self.tau, self.eps = heads, dim, vdim, decay_rank, tau, eps
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.in_proj = mk(2 * heads * dim + 2 * heads * vdim + decay_rank, width)      # rows: q | k | v | g | a1
        self.a2, self.a2_bias = mk(heads * dim, decay_rank), f32(heads * dim)
        self.norm = f32(vdim)
        self.o = mk(width, heads * vdim)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"rec": ((self.heads, self.dim, self.vdim), torch.float32)}

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        N, H, D, V = B * S, self.heads, self.dim, self.vdim
        p = F.linear(h, self.in_proj)
        q, k = p[..., :H * D].unflatten(-1, (H, D)), p[..., H * D:2 * H * D].unflatten(-1, (H, D))
        v = p[..., 2 * H * D:2 * H * D + H * V].unflatten(-1, (H, V))
        g = p[..., 2 * H * D + H * V:2 * H * D + 2 * H * V].reshape(N * H, V)
        z = F.linear(p[..., 2 * H * D + 2 * H * V:], self.a2)
        o = seqmix.gla_scan(q, k, v, z, self.a2_bias, self.tau, st["rec"], ctx.slots, ctx.lens, ctx.fresh)       # float [B,S,H,V]
        on = seqmix.rms_norm(o.view(N * H, V), self.norm, self.eps, gate=g, out_dtype=h.dtype)
        return F.linear(on.view(N, H * V), self.o).view(B, S, -1)
