"""Replay of a recorded serving trace: token ids are fed step by step through a serving model's own step function and state
manager, and the logits at the asked positions are written out; nothing is sampled.  Used by ``bin/trace_run`` to compare runs
(other batch compositions, other cuts of the same requests, other builds) position by position.

One input line per step: ``{"step": n, "entries": [{"id", "tokens", "want"}...], "end": [ids]}``.  The entries of a step are one
right-padded batch; they either all start (a slot is taken for each) or all continue by one token.  ``want`` indexes into the
entry's tokens of this step.  Requests named in ``end`` give their slots back after the step."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List

import numpy as np
import torch


class TraceReplayer:
    def __init__(self, model, out_dir: str):
        if not hasattr(model, "forward_step"):
            raise TypeError(f"{type(model).__name__} has no slot-based step function (forward_step / logits / states)")
        self.model, self.out_dir = model, out_dir
        self.slot_of: Dict[str, int] = {}

    @torch.no_grad()
    def step(self, rec: dict) -> None:
        m, mgr = self.model, self.model.states
        entries = rec["entries"]
        if entries:
            ids = [e["id"] for e in entries]
            starting = [i not in self.slot_of for i in ids]
            if any(starting) != all(starting):
                raise ValueError("a step either starts all of its requests or continues all of them")
            fresh = all(starting)
            if fresh:
                for i in ids:
                    self.slot_of[i] = mgr.alloc()
            lens = [len(e["tokens"]) for e in entries]
            if min(lens) < 1:
                raise ValueError("an entry without tokens")
            dev = next(m.parameters()).device
            tokens = torch.zeros(len(entries), max(lens), dtype=torch.long)
            for b, e in enumerate(entries):
                tokens[b, : lens[b]] = torch.tensor(e["tokens"], dtype=torch.long)
            slots = [self.slot_of[i] for i in ids]
            pos0 = [mgr.length[s] for s in slots]
            x = m.forward_step(tokens.to(dev), lens, slots, pos0, fresh)
            mgr.advance(slots, lens)
            rows = [(b, t) for b, e in enumerate(entries) for t in e.get("want", [])]
            if rows:
                bi = torch.tensor([r[0] for r in rows], device=dev)
                ti = torch.tensor([r[1] for r in rows], device=dev)
                logits = m.logits(x[bi, ti]).float().cpu().numpy().astype("<f4")
                path = os.path.join(self.out_dir, f"{rec['step']}.f32")
                with open(path + ".part", "wb") as f:
                    f.write(np.ascontiguousarray(logits).tobytes())
                os.replace(path + ".part", path)
        for i in rec.get("end", []):
            if i in self.slot_of:
                mgr.free(self.slot_of.pop(i))

    def run(self, lines: Iterable[str], out) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            self.step(rec)
            out.write(f"done {rec['step']}\n")
            out.flush()
