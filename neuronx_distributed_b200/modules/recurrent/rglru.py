"""Recurrent block with a real-gated linear recurrent unit (the recurrent block of Griffin: De et al., "Griffin: Mixing Gated
Linear Recurrences with Local Attention for Efficient Language Models").  Two branches of ``rwidth`` channels:
``y = gelu_tanh(W_y h + b)`` and ``u = conv(W_x h + b)`` (short causal convolution with bias).  Per channel, with block-diagonal gate
matrices, ``r = sigmoid(R u + b_r)``, ``i = sigmoid(I u + b_i)``, ``a = exp(-8 r softplus(lam))``,
``s_t = a s_(t-1) + sqrt(1 - a^2) i u_t`` and the block returns ``W_o (s * y)``.  The gates, decays and the state are float: the
gate products are batched matrix products of the convolution output with the gate matrices as stored, accumulated in float."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix
from ..short_conv import ShortConv


class RealGatedLRUBlock(nn.Module):
    def __init__(self, width: int, rwidth: int, blocks: int, taps: int, dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        assert rwidth % blocks == 0, "the recurrent width must divide into the gate blocks"
        self.rwidth, self.blocks, self.dtype = rwidth, blocks, dtype
        wb = rwidth // blocks
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.in_proj, self.in_bias = mk(2 * rwidth, width), mk(2 * rwidth)             # rows: y | x
        self.conv = ShortConv(rwidth, taps, bias=True, residual=False, device=device)
        self.gate_r, self.gate_i = mk(blocks, wb, wb), mk(blocks, wb, wb)              # stored transposed: [block, in, out]
        self.gate_r_bias, self.gate_i_bias = f32(rwidth), f32(rwidth)
        self.lam_softplus = f32(rwidth)                                                # softplus(lam), formed once in float
        self.o = mk(width, rwidth)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"conv": self.conv.state_spec(self.dtype), "rec": ((self.rwidth,), torch.float32)}

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        N, W = B * S, self.rwidth
        yx = F.linear(h, self.in_proj, self.in_bias)
        u = self.conv(yx[..., W:], st["conv"], ctx, h.dtype)                            # [B,S,W]
        ub = u.view(N, self.blocks, W // self.blocks).transpose(0, 1)                   # [blocks, N, wb]
        # gate pre-activations in float: products of the activations with the gate matrices as they are stored, float accumulation
        gr, gi = seqmix.matmul_f32(ub, self.gate_r), seqmix.matmul_f32(ub, self.gate_i)
        out = seqmix.rglru_scan(u, gr, gi, self.gate_r_bias, self.gate_i_bias, self.lam_softplus, yx[..., :W], st["rec"], ctx.slots,
                                ctx.lens, ctx.fresh)
        return F.linear(out, self.o)
