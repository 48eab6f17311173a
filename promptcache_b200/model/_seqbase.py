"""Shared plumbing of the models that run a batch of sequences over a `SlotPool`: the step function, the HF-style
single-sequence `forward` the `GenerationEngine` drives, CUDA-graph replay of the decode step.

A subclass sets `width`, `vocab_size`, `compute_dtype`, `state_specs()` and implements `_layers(ids, batch, rows)`, which
runs the concatenated tokens of the batch through its layers and returns float32 logits of the token rows `rows`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import _native_seq as nsq
from ._kv import CausalLMOutput
from ._state import SeqState, SlotPool


class SlotPoolCausalLM(nn.Module):
    accepts_max_position = True   # forward() takes (and ignores) the host-known max position id: positions are row counts
    full_position_ids = False
    uses_slot_pool = True

    def _init_runtime(self, device, max_tokens: Optional[int] = None):
        self._device = torch.device(device)
        self.pool = SlotPool(self.state_specs(), self.compute_dtype, self._device, max_tokens=max_tokens)
        self.use_cuda_graphs = True
        self._graphs = {}
        self._graph_seen = {}
        self.max_graphs = 8
        self.layer_trace = None  # a list: the residual stream after every layer is appended (debugging, tests)

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def dtype(self) -> torch.dtype:
        return self.compute_dtype

    def set_max_tokens(self, max_tokens: Optional[int]) -> None:
        self.pool = SlotPool(self.state_specs(), self.compute_dtype, self._device, max_tokens=max_tokens)
        self._graphs.clear()

    def new_sequence(self) -> SeqState:
        return SeqState(self.pool)

    # ---- the step ---------------------------------------------------------------------------------------------
    @torch.inference_mode()
    def step(self, entries: Sequence[Tuple[SeqState, Sequence[int]]], want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Run the next tokens of several sequences as ONE batch: `entries` = [(sequence, its next token ids)], `want[b]` =
        the places among entry b's tokens whose logits are asked for (default: the last one).  Returns float32
        [number of wanted places, vocab] in the order of the entries and of `want`.  The sequences' states advance."""
        if not entries:
            return torch.zeros(0, self.vocab_size, dtype=torch.float32, device=self._device)
        lens = [len(toks) for _, toks in entries]
        if min(lens) <= 0:
            raise ValueError("every entry of a step needs at least one token")
        if len({id(s) for s, _ in entries}) != len(entries):
            raise ValueError("a sequence may appear once in a step")
        for (seq, _), n in zip(entries, lens):
            if seq.pool is not self.pool or seq.slot is None:
                raise ValueError("a sequence of another pool (or a freed one) was passed to step()")
            self.pool.reserve(seq.slot, seq.rows + n)
        slots = [s.slot for s, _ in entries]
        pos0 = [s.rows for s, _ in entries]
        rows, off = [], 0
        for b, n in enumerate(lens):
            w = [n - 1] if want is None else list(want[b])
            for i in w:
                if not 0 <= i < n:
                    raise ValueError(f"wanted place {i} is outside the {n} tokens of entry {b}")
                rows.append(off + i)
            off += n
        flat = [int(t) for _, toks in entries for t in toks]
        prev = []   # every token's predecessor in its own sequence (-1: none)
        for seq, toks in entries:
            prev += [seq.last_token if seq.rows > 0 else -1] + [int(t) for t in list(toks)[:-1]]
        parity = [s.steps & 1 for s, _ in entries]
        decode = max(lens) == 1 and min(pos0) > 0 and len(rows) == len(entries)
        logits = None
        if decode and self.use_cuda_graphs and not torch.cuda.is_current_stream_capturing():
            logits = self._decode_replay(flat, slots, pos0, prev, parity)
        if logits is None:
            batch = nsq.Batch(slots, pos0, lens, self._device, parity)
            both = torch.tensor(flat + prev, dtype=torch.int64).pin_memory().to(self._device, non_blocking=True)
            ids, batch.prev_ids = both[:len(flat)], both[len(flat):]
            rows_t = torch.tensor(rows, dtype=torch.int32).pin_memory().to(self._device, non_blocking=True) if rows else None
            logits = self._layers(ids, batch, rows_t)
        for (seq, toks), n in zip(entries, lens):
            self.pool.rows[seq.slot] += n
            seq.steps += 1
            seq.last_token = int(toks[-1])
        return logits

    def _decode_replay(self, flat, slots, pos0, prev, parity):
        """One-token-per-sequence steps of a given batch size replay ONE captured graph: everything that changes from step
        to step (token ids, slots, positions) lives in static device buffers the kernels read at run time."""
        B = len(flat)
        key = (B, self.pool.version)
        entry = self._graphs.get(key)
        if entry is None:
            self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
            if self._graph_seen[key] < 2:
                return None  # the first such step runs eagerly (it also warms up the libraries' workspaces)
            if len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            batch = nsq.Batch(slots, pos0, [1] * B, self._device, parity)
            both = torch.tensor(flat + prev, dtype=torch.int64, device=self._device)
            ids, batch.prev_ids = both[:B], both[B:]
            rows_t = torch.arange(B, dtype=torch.int32, device=self._device)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = nsq.launch_count()
            with torch.cuda.graph(graph):  # recording only: no kernel runs, no state advances
                out = self._layers(ids, batch, rows_t)
            # every tensor the recorded kernels read must outlive the graph: the row list too
            entry = (graph, batch, both, out, nsq.launch_count() - before, rows_t)
            self._graphs[key] = entry
        graph, batch, both, out, n_native = entry[:5]
        ar = list(range(B))
        host = torch.tensor(ar + list(pos0) + list(slots) + list(pos0) + [1] * B + ar + list(parity), dtype=torch.int32)
        batch.meta.copy_(host.pin_memory(), non_blocking=True)
        both.copy_(torch.tensor(flat + prev, dtype=torch.int64).pin_memory(), non_blocking=True)
        graph.replay()
        nsq.note_replayed_launches(n_native)
        return out.clone()

    # ---- the single-sequence interface of the generation engine --------------------------------------------------
    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor = None, position_ids: Optional[torch.Tensor] = None, past_key_values=None,
                attention_mask=None, use_cache: Optional[bool] = None, max_position: Optional[int] = None,
                static_logits_ok: bool = False, **_):
        """`past_key_values` is the `SeqState` an earlier call returned (None starts a sequence).  Positions are the
        sequence's own token count, so `position_ids` is not read.  The logits of the LAST token only are returned, shaped
        [1, 1, vocab], which is all a generation loop reads."""
        if input_ids is None or input_ids.dim() != 2 or input_ids.shape[0] != 1:
            raise ValueError("slot-pool models take input_ids of shape [1, q]; batches go through step()")
        if not input_ids.is_cuda:
            raise nsq.NativeError("promptcache_b200 models run on CUDA only (no CPU fallback)")
        seq = past_key_values if past_key_values is not None else self.new_sequence()
        if not isinstance(seq, SeqState):
            raise ValueError("past_key_values must be the SeqState handle a previous forward returned")
        logits = self.step([(seq, input_ids[0].tolist())])
        return CausalLMOutput(logits.view(1, 1, -1), seq)

    def _layers(self, ids: torch.Tensor, batch, rows: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError
