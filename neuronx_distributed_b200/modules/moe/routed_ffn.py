"""Routed feed-forward with independent (non-normalised) expert weights and plain two-matrix experts, for serving:
scores ``s = act(W_router h)`` in float (the framework's ``RouterTopK``; sigmoid here), the ``top`` largest are chosen, the output
is ``sum_e s_e * scale * expert_e(h)`` plus an always-on shared expert.  Experts are ``W_down act(W_up h)`` without biases or
gating, kept as stacks ``[E, ff, width]`` / ``[E, width, ff]``.

Two execution shapes, both summing the chosen experts in float (``moe_combine``):
* few rows (token generation): the chosen experts' matrices are streamed once by ``indexed_gemv`` — no host synchronisation;
* many rows (prompts): rows are sorted by expert and every non-empty expert runs two dense matrix products."""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix
from .routing import RouterTopK


class RoutedFFN(nn.Module):
    small_batch_rows = 64          # up to this many (row, expert) pairs the streaming path is used

    def __init__(self, width: int, ff: int, experts: int, top: int, weight_scale: float = 1.0, shared_ff: int = 0,
                 router_act: str = "sigmoid", dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        self.width, self.ff, self.experts, self.top, self.weight_scale, self.shared_ff = width, ff, experts, top, weight_scale, shared_ff
        self.router = RouterTopK(experts, top, width, dtype=torch.float32, device=device, act_fn=router_act)
        self.router.requires_grad_(False)
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        self.up, self.down = mk(experts, ff, width), mk(experts, width, ff)
        if shared_ff:
            self.shared_up, self.shared_down = mk(shared_ff, width), mk(width, shared_ff)

    def route(self, h: torch.Tensor):
        """Float scores of all experts → (weights ``[N, top]`` float, expert ids ``[N, top]``)."""
        scores = self.router.apply_activation_fn(self.router.get_router_logits(h))
        w, idx = torch.topk(scores, self.top, dim=-1)
        return w * self.weight_scale, idx

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """``h [N, width]`` → ``[N, width]``."""
        N = h.shape[0]
        w, idx = self.route(h)
        M = N * self.top
        if M <= self.small_batch_rows:
            sel = idx.reshape(-1).to(torch.int32)
            mid = seqmix.indexed_gemv(self.up, sel, h.repeat_interleave(self.top, 0), True)
            eo = seqmix.indexed_gemv(self.down, sel, mid, False)
            src = torch.arange(M, device=h.device, dtype=torch.int32).view(N, self.top)
        else:
            flat = idx.reshape(-1)
            order = torch.argsort(flat, stable=True)
            counts = torch.bincount(flat, minlength=self.experts).tolist()
            xs = h[order // self.top]
            eo = torch.empty(M, self.width, dtype=h.dtype, device=h.device)
            off = 0
            for e, c in enumerate(counts):
                if c:
                    eo[off:off + c] = F.linear(seqmix.gelu_erf(F.linear(xs[off:off + c], self.up[e])), self.down[e])
                    off += c
            src = torch.empty(M, dtype=torch.int32, device=h.device)
            src[order] = torch.arange(M, device=h.device, dtype=torch.int32)
            src = src.view(N, self.top)
        base = F.linear(seqmix.gelu_erf(F.linear(h, self.shared_up)), self.shared_down) if self.shared_ff else None
        return seqmix.moe_combine(eo, src, w.contiguous(), base)
