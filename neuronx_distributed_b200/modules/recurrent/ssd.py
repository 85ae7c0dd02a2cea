"""Selective state space mixer with a scalar decay per head (Dao, Gu, "Transformers are SSMs: Generalized Models and Efficient
Algorithms Through Structured State Space Duality").  One input projection gives ``[z | x | B | C | dt]`` with
``inner = heads * vdim`` channels for z and x, ``groups * state`` for B and C and one step size per head.  x, B and C pass a short
causal convolution (with bias) and silu; ``dt = softplus(dt + dt_bias)`` without clamping; per head (reading its group's B and C)
``M_t = exp(-exp(A_log) dt) M_(t-1) + dt B_t x_t^T`` with ``M [state, vdim]`` float and ``y_t = M_t^T C_t + D x_t``.  The output
is gated FIRST, ``y * silu(z)``, then RMS-normed in ``norm_groups`` equal parts, weighted and projected out.

The step sizes come from their own float-accumulated product (they enter the recurrence); state per sequence: the convolution
history and the float memory."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix
from ..short_conv import ShortConv


class SelectiveStateSpace(nn.Module):
    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, norm_groups: int, taps: int, eps: float = 1e-6,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        assert heads % groups == 0 and (heads * vdim) % norm_groups == 0
        self.heads, self.vdim, self.state, self.groups, self.norm_groups = heads, vdim, state, groups, norm_groups
        self.eps, self.dtype = eps, dtype
        self.inner = heads * vdim
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.in_proj = mk(2 * self.inner + 2 * groups * state, width)                # rows: z | x | B | C
        self.dt_proj = mk(heads, width)
        self.conv = ShortConv(self.inner + 2 * groups * state, taps, bias=True, residual=False, device=device)
        self.a_log, self.dt_bias, self.d_skip = f32(heads), f32(heads), f32(heads)
        self.norm = f32(self.inner)
        self.o = mk(width, self.inner)

    @property
    def out_features(self) -> int:
        return self.inner

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"conv": self.conv.state_spec(self.dtype), "rec": ((self.heads, self.state, self.vdim), torch.float32)}

    def mix(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor], out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        B, S, W = h.shape
        N, H, V, G, Ns, I = B * S, self.heads, self.vdim, self.groups, self.state, self.inner
        p = F.linear(h, self.in_proj)
        c = self.conv(p[..., I:], st["conv"], ctx, h.dtype, silu=True)               # [B,S,x|B|C]
        x = c[..., :I].unflatten(-1, (H, V))
        bm, cm = c[..., I:I + G * Ns].unflatten(-1, (G, Ns)), c[..., I + G * Ns:].unflatten(-1, (G, Ns))
        dt = seqmix.linear_f32(h.view(N, W), self.dt_proj).view(B, S, H)
        y = seqmix.ssd_scan(x, bm, cm, dt, self.a_log, self.dt_bias, self.d_skip, st["rec"], ctx.slots, ctx.lens, ctx.fresh)
        return seqmix.group_rms_norm_gated(y.view(N, I), p.view(N, -1)[:, :I], self.norm, self.norm_groups, self.eps, True, out, out_scale)

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        heads = torch.empty(B * S, self.out_features, dtype=h.dtype, device=h.device)
        return F.linear(self.mix(h, ctx, st, heads), self.o).view(B, S, -1)
