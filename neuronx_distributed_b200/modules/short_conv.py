"""Short causal convolution over time, one filter per channel, with the last ``taps - 1`` inputs of every sequence carried as state
(``csrc/seqmix/short_conv.cu``).  Two uses: the residual input convolution of a sublayer (``h + conv(h)``, no bias) and the plain
convolution inside a recurrent block (``conv(h) + bias``)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import nn

from ..ops import seqmix


class ShortConv(nn.Module):
    def __init__(self, channels: int, taps: int, bias: bool = False, residual: bool = False, device=None):
        super().__init__()
        self.channels, self.taps, self.residual = channels, taps, residual
        self.weight = nn.Parameter(torch.zeros(channels, taps, dtype=torch.float32, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(channels, dtype=torch.float32, device=device), requires_grad=False) if bias else None

    def state_spec(self, in_dtype: torch.dtype) -> Tuple[Tuple[int, ...], torch.dtype]:
        """Per-sequence state: the last ``taps - 1`` inputs, in the dtype the convolution reads."""
        return (self.taps - 1, self.channels), in_dtype

    def forward(self, x: torch.Tensor, state: torch.Tensor, ctx, out_dtype: torch.dtype, silu: bool = False) -> torch.Tensor:
        """``x [B,S,C]`` (last dim contiguous) → ``[B,S,C]`` (``silu`` applied when asked); ``state`` is updated in place for the
        rows' slots."""
        return seqmix.short_conv(x, self.weight, self.bias, state, ctx.slots, ctx.lens, ctx.fresh, self.residual, out_dtype, silu)
