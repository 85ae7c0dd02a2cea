"""Latent (compressed key/value) attention with rotary positions on a separate key part and a sliding window.

Per token the layer keeps only a normalised latent ``c`` (``kv_rank`` numbers) and ONE rotated key part shared by all heads
(``rot_dim`` numbers).  Queries go through their own latent.  A head's score against position j is
``(q_unrot . W_uk c_j + q_rot . k_rot_j) * scale``; it is evaluated in the absorbed form ``(W_uk^T q_unrot) . c_j`` so that
neither keys nor values are ever expanded: the attention kernel returns the weighted sum of latents and ``W_uv`` is applied
afterwards.  Position i sees ``i - window < j <= i``, so the cache is a ring of ``window`` rows per sequence
(``csrc/seqmix/latent_attention.cu``).  A prompt that starts a sequence attends over its own prepared rows and leaves its last
``window`` rows in the ring; later single tokens append to the ring and attend over it."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class LatentWindowAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, window: int,
                 scale: float, rot_base: float, rot_dims: int, eps: float, dtype: torch.dtype = torch.bfloat16, device=None,
                 max_seq_len: int = 1 << 30, block_products: bool = True, query_block: int = 128):
        super().__init__()
        self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank, self.q_rank = heads, dim, rot_dim, vdim, kv_rank, q_rank
        self.window, self.scale, self.rot_dims, self.eps, self.dtype = window, scale, rot_dims, eps, dtype
        self.ring = max(1, min(window, max_seq_len))
        self.block_products, self.query_block = block_products, query_block
        self.max_seq_len = max_seq_len
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.ones(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.dq, self.dq_norm, self.uq = mk(q_rank, width), f32(q_rank), mk(heads * (dim + rot_dim), q_rank)
        self.dkv, self.dkv_norm = mk(kv_rank + rot_dim, width), f32(kv_rank)
        self.uk, self.uv = mk(heads, dim, kv_rank), mk(heads, vdim, kv_rank)          # per head [out, in]
        self.o = mk(width, heads * vdim)
        self.register_buffer("inv_freq", seqmix.rotary_inv_freq(rot_dims, rot_base, device), persistent=False)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"kv": ((self.ring, self.kv_rank + self.rot_dim), self.dtype)}

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        N, H, D, R = B * S, self.heads, self.dim, self.rot_dim
        cq = seqmix.rms_norm(F.linear(h.view(N, -1), self.dq), self.dq_norm, self.eps)
        q = F.linear(cq, self.uq).view(B, S, H, D + R)
        kv = F.linear(h, self.dkv)
        rows = seqmix.latent_kv_store(kv, self.dkv_norm, self.eps, self.inv_freq, self.rot_dims, ctx.pos0, ctx.lens, ctx.slots, st["kv"],
                                      want_rows=ctx.fresh)
        seqmix.rope_q_(q, D, self.rot_dims, self.inv_freq, ctx.pos0)
        qa = torch.bmm(q.view(N, H, D + R)[:, :, :D].transpose(0, 1), self.uk)                       # [H,N,D] @ [H,D,C]
        if self.block_products:
            o = self._attend_products(qa, q, rows, ctx, st)
        elif ctx.fresh:
            o = seqmix.latent_window_attention(qa, q, D, rows, None, ctx.pos0, ctx.lens, self.window, self.scale)
        else:
            o = seqmix.latent_window_attention(qa, q, D, st["kv"], ctx.slots, ctx.pos0, ctx.lens, self.window, self.scale)
        ov = torch.bmm(o, self.uv.transpose(1, 2))                                                     # [H,N,C] @ [H,C,V]
        return F.linear(ov.transpose(0, 1).reshape(N, H * self.vdim), self.o).view(B, S, -1)

    def _attend_products(self, qa: torch.Tensor, q: torch.Tensor, rows, ctx, st) -> torch.Tensor:
        """Scores and weighted sums as matrix products with the heads folded into the row dimension (all heads share the keys):
        a prompt is cut into blocks of ``query_block`` tokens, each multiplied with the ``query_block + window - 1`` key rows it can
        see; a single token multiplies its sequence's ring.  The softmax over the visible keys runs in float in between
        (``window_softmax``).  Returns ``[H, N, C]``."""
        B, S, H, _ = q.shape
        C, R, D = self.kv_rank, self.rot_dim, self.dim
        qcat = torch.cat([qa.view(H, B, S, C).permute(1, 2, 0, 3), q[..., D:]], -1)                   # [B,S,H,C+R]
        if not ctx.fresh:
            kc = st["kv"].index_select(0, ctx.slots.long())                                            # [B,ring,C+R]
            sc = seqmix.matmul_f32(qcat.view(B, H, C + R), kc.transpose(1, 2))                         # [B,H,ring]
            p = seqmix.window_softmax(sc, self.scale, True, H, 1, 1, 1, self.window, ctx.pos0, ctx.lens, q.dtype)
            return torch.bmm(p, kc[..., :C]).transpose(0, 1).contiguous()                              # [H,B,C]
        Qb = min(self.query_block, S)
        nblk = -(-S // Qb)
        Sp, w = nblk * Qb, min(self.window, S)
        span = Qb + w - 1
        qp = F.pad(qcat, (0, 0, 0, 0, 0, Sp - S)).view(B * nblk, Qb * H, C + R)
        kp = F.pad(rows, (0, 0, w - 1, Sp - S)).unfold(1, span, Qb)                                    # [B,nblk,C+R,span] view
        kt = kp.reshape(B * nblk, C + R, span)
        sc = seqmix.matmul_f32(qp, kt).view(B, nblk, Qb * H, span)
        p = seqmix.window_softmax(sc, self.scale, False, H, Qb, nblk, w, self.window, ctx.pos0, ctx.lens, q.dtype)
        o = torch.bmm(p.view(B * nblk, Qb * H, span), kt[:, :C].transpose(1, 2))                       # [B*nblk, Qb*H, C]
        return o.view(B, Sp, H, C)[:, :S].permute(2, 0, 1, 3).reshape(H, B * S, C)
