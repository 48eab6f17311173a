"""Batch engine: the scheduler of the slot-pool models.

Requests are identified by a caller-chosen id.  `step` runs the next tokens of several requests as one batch through the
model's own step function (`SlotPoolCausalLM.step`) and hands back the logits that were asked for; `end` gives a
request's slot back to the pool.  `generate` is the batched counterpart of `GenerationEngine.generate`: requests are
admitted in waves that fit the token budget, a wave's prompts are prefilled as one batch and then decoded together, one
token per request and step, a request leaving the batch when it stops; sampling uses the same `GenerationParameters`
(temperature, top-p, top-k, repetition penalty) as the single-sequence engine.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .generation_engine import GenerationParameters
from .model._state import SeqState


class BatchEngine:
    def __init__(self, model, max_tokens: Optional[int] = None):
        if not getattr(model, "uses_slot_pool", False):
            raise TypeError("BatchEngine schedules slot-pool models; the prompt-cache models are served by CacheEngine + GenerationEngine")
        self.model = model
        if max_tokens is not None:
            model.set_max_tokens(max_tokens)
        self.max_tokens = max_tokens
        self.live: Dict[str, SeqState] = {}

    def tokens_held(self) -> int:
        return sum(s.rows for s in self.live.values())

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Optional[Sequence[int]]]], end: Sequence[str] = ()) -> torch.Tensor:
        """entries: (request id, its next tokens, places among them whose logits are wanted or None for the last one).
        A request id that is not live starts a new sequence.  Returns float32 [wanted, vocab]."""
        batch, want = [], []
        for rid, toks, w in entries:
            seq = self.live.get(rid)
            if seq is None:
                seq = self.live[rid] = self.model.new_sequence()
            batch.append((seq, toks))
            want.append([len(toks) - 1] if w is None else list(w))
        if self.max_tokens is not None:
            held = self.tokens_held() + sum(len(t) for _, t in batch)
            if held > self.max_tokens:
                raise ValueError(f"the step would hold {held} tokens, more than the engine's budget of {self.max_tokens}")
        logits = self.model.step(batch, want)
        for rid in end:
            self.end(rid)
        return logits

    def end(self, rid: str) -> None:
        seq = self.live.pop(rid, None)
        if seq is not None:
            seq.free()

    # ---- batched generation --------------------------------------------------------------------------------------
    def _sample(self, logits: torch.Tensor, params: GenerationParameters, history: List[List[int]], procs) -> List[int]:
        greedy = params.temperature < 1e-5 or params.top_p < 1e-8
        if greedy and params.repetition_penalty <= 1.0:
            return torch.argmax(logits, dim=-1).tolist()   # one device-to-host read for the whole batch
        out = []
        for b in range(logits.shape[0]):
            ctx = torch.as_tensor([history[b]], device=logits.device) if params.repetition_penalty > 1.0 else None
            row = procs(ctx, logits[b:b + 1])[0]
            out.append(int(torch.argmax(row)) if greedy else int(torch.multinomial(torch.softmax(row, dim=-1), num_samples=1)))
        return out

    @torch.inference_mode()
    def generate(self, prompts: Sequence[Sequence[int]], params: GenerationParameters) -> List[List[int]]:
        """New token ids per prompt (a stop token ends a request and is kept, as in the single-sequence engine)."""
        procs = params.get_logits_processor()
        results: List[List[int]] = [[] for _ in prompts]
        todo = list(range(len(prompts)))
        serial = 0
        while todo:
            wave, held = [], self.tokens_held()
            while todo:  # admit while the wave's worst-case footprint fits the budget
                need = len(prompts[todo[0]]) + params.max_new_tokens
                if self.max_tokens is not None and wave and held + need > self.max_tokens:
                    break
                held += need
                wave.append(todo.pop(0))
            names = {i: f"gen{serial}-{i}" for i in wave}
            serial += 1
            active = list(wave)
            history = {i: list(prompts[i]) for i in wave}
            logits = self.step([(names[i], list(prompts[i]), None) for i in active])
            for _ in range(params.max_new_tokens):
                toks = self._sample(logits, params, [history[i] for i in active], procs)
                nxt = []
                for i, t in zip(active, toks):
                    results[i].append(t)
                    history[i].append(t)
                    if t in params.stop_token_ids or len(results[i]) >= params.max_new_tokens:
                        self.end(names[i])
                    else:
                        nxt.append((i, t))
                if not nxt:
                    break
                active = [i for i, _ in nxt]
                logits = self.step([(names[i], [t], None) for i, t in nxt])
            for i in wave:
                self.end(names[i])
        return results
