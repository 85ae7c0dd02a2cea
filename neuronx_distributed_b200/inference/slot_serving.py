"""Serving wrapper shared by the model families whose layers keep per-sequence state in slots (``state_cache.py``): the step
function over any rows and slots (``forward_step`` → float residual stream, ``logits``), and on top of it the static-batch entry
points of ``LlamaForInference`` (``context_encoding`` / ``token_generation`` / ``generate``) with the framework's sampler.

A family provides a language model with ``embed`` (a parameter, for the device), ``state_specs()``,
``body(input_ids, ctx, states, tap)`` → float ``[B,S,width]`` and ``logits(rows)``; the subclass adds ``from_pretrained`` and
``load_checkpoint_tensors``."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..utils.sampling import Sampler
from .state_cache import SequenceStateManager, StepContext


class SlotServingModel(nn.Module):
    def __init__(self, cfg, lm: nn.Module, batch_size: int = 1, max_seq_len: int = 2048, on_device_sampling: bool = True,
                 sampler: Optional[Sampler] = None):
        super().__init__()
        self.cfg = cfg
        self.lm = lm
        self.batch_size, self.max_seq_len = batch_size, max_seq_len
        self.states = SequenceStateManager(self.lm.state_specs(), num_slots=max(batch_size, 1), device=cfg.device)
        self.sampler = sampler or Sampler(top_k=1, vocab_parallel=False)
        self.on_device_sampling = on_device_sampling
        self._rows = None

    def load_checkpoint_tensors(self, sd) -> None:
        raise NotImplementedError

    def load_state_dict(self, sd, strict: bool = True):
        if "embed" in sd and "final.norm" in sd:
            return self.load_checkpoint_tensors(sd)
        return self.lm.load_state_dict(sd, strict=strict)

    def state_dict(self, *a, **k):
        return self.lm.state_dict(*a, **k)

    # ---- the step function: any rows, any slots --------------------------------------------------------------------------------
    def _i32(self, v) -> torch.Tensor:
        if isinstance(v, torch.Tensor):
            return v.to(device=self.lm.embed.device, dtype=torch.int32)
        return torch.tensor(list(v), dtype=torch.int32, device=self.lm.embed.device)

    @torch.no_grad()
    def forward_step(self, input_ids: torch.Tensor, lens, slots, pos0, fresh: bool, tap=None) -> torch.Tensor:
        """``input_ids [B,S]`` (right-padded), ``lens / slots / pos0 [B]`` → float residual stream ``[B,S,width]`` after the last
        layer.  ``fresh``: the rows start new sequences (prompts); otherwise they continue from their slots' state."""
        if not fresh and input_ids.shape[1] != 1:
            raise ValueError("a continuing step carries one token per row")
        ctx = StepContext(self._i32(lens), self._i32(slots), self._i32(pos0), bool(fresh))
        return self.lm.body(input_ids, ctx, self.states, tap)

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        return self.lm.logits(rows)

    def _pick(self, logits: torch.Tensor) -> torch.Tensor:
        return self.sampler.sample(logits) if self.on_device_sampling else logits

    # ---- static-batch entry points (rows ↔ slots held for the lifetime of the batch) ---------------------------------------------
    def _batch_rows(self, B: int):
        """Slots of the static batch and the constant step tensors that go with it, made once (nothing is copied from the host in
        a token-generation step, so the step can be captured in a CUDA graph)."""
        if self._rows is None or len(self._rows[0]) != B:
            for s in (self._rows[0] if self._rows else []):
                self.states.free(s)
            slots = [self.states.alloc() for _ in range(B)]
            dev = self.lm.embed.device
            self._rows = (slots, torch.tensor(slots, dtype=torch.int32, device=dev), torch.ones(B, dtype=torch.int32, device=dev),
                          torch.zeros(B, dtype=torch.int32, device=dev), torch.arange(B, device=dev))
        return self._rows

    @torch.no_grad()
    def context_encoding(self, input_ids: torch.Tensor, last_token_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``input_ids [B,S]`` right-padded prompts → next token ids ``[B]`` (or logits)."""
        B, S = input_ids.shape
        _, slots, _, zeros, rows = self._batch_rows(B)
        last = last_token_index if last_token_index is not None else torch.full((B,), S - 1, device=input_ids.device)
        x = self.forward_step(input_ids, last + 1, slots, zeros, True)
        return self._pick(self.logits(x[rows, last.long()]))

    @torch.no_grad()
    def token_generation(self, input_ids: torch.Tensor, positions: torch.Tensor, kv_len: Optional[int] = None) -> torch.Tensor:
        """``input_ids [B,1]``, ``positions [B]`` → next token ids ``[B]`` (or logits)."""
        _, slots, ones, _, _ = self._batch_rows(input_ids.shape[0])
        x = self.forward_step(input_ids, ones, slots, positions, False)
        return self._pick(self.logits(x[:, 0]))

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int, prompt_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S = prompt_ids.shape
        lens = prompt_lens if prompt_lens is not None else torch.full((B,), S, device=prompt_ids.device, dtype=torch.long)
        tok = self.context_encoding(prompt_ids, lens - 1)
        out, pos = [tok], lens.clone()
        for _ in range(max_new_tokens - 1):
            tok = self.token_generation(tok.view(B, 1), pos)
            out.append(tok)
            pos = pos + 1
        return torch.stack(out, dim=1)
