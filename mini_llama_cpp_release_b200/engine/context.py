"""A context: one model's cache on one device, and the step function over it.

The reference's context is one sequence: its cache, its position, its token history
(include/mini_llama/context.h:11-30), and `forward_batch(model, ctx, batch)` feeds it
(src/batch.cpp:33-52).  Here a context holds many sequences, each in a slot; a step
brings the next tokens of some of them, runs exactly those tokens as one batch against
the cache, and returns logits at the places asked for.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels
from ..cache.paged import PAGE_SIZE, PagedCache
from .batch import MiniBatch, SequenceChunk
from .decode_runner import DecodeRunner
from .model import Model
from .step_info import StepInfo


class ContextOverflow(ValueError):
    """A sequence would pass the model's largest position."""


class Context:
    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None, page_size: int = PAGE_SIZE):
        """`max_tokens`: the most tokens live sequences hold at any time, each sequence's
        count rounded up to whole pages of `page_size` tokens."""
        self.model = model
        rt = model.runtime
        if max_seqs is None:
            max_seqs = min((max_tokens + page_size - 1) // page_size, 4096)
        with torch.cuda.device(rt.device):
            self.cache = PagedCache(model.cache_needs(), model.reads_cache_of(), model.state_specs(), max_tokens,
                                    max_seqs, rt.dtype, rt.device, page_size)
        self.max_position = model.config.max_position_embeddings
        self.token_history: Dict[int, List[int]] = {}
        self.n_steps = 0
        self._pinned: Optional[torch.Tensor] = None            # host staging buffer of `describe`
        # decoding through captured graphs needs every part to be free of host round trips
        self.use_graphs = all(getattr(p, "graph_safe", False) for p in model.graph_relevant_parts())
        self._runners: Dict[tuple, DecodeRunner] = {}

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        slot = self.cache.acquire()
        self.token_history[slot] = []
        return slot

    def release(self, slot: int) -> None:
        self.cache.release(slot)
        self.token_history.pop(slot, None)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ------------------------------------------------------------------ the step
    def describe(self, batch: MiniBatch) -> StepInfo:
        """Reserve pages for the batch's tokens and put its description on the device."""
        cache = self.cache
        tokens: List[int] = []
        positions: List[int] = []
        tok_seq: List[int] = []
        cu = [0]
        start_pos: List[int] = []
        slots: List[int] = []
        want_rows: List[int] = []
        max_q = max_kv = 0
        for c in batch.chunks:
            if c.slot not in cache.length:
                raise ValueError(f"forward_batch: slot {c.slot} is not held")
            start = cache.length[c.slot]
            if start + len(c.tokens) > self.max_position:
                raise ContextOverflow(
                    f"slot {c.slot}: {start} cached + {len(c.tokens)} new tokens pass max_position_embeddings "
                    f"{self.max_position}")                                          # src/forward.cpp:23-25
        for c in batch.chunks:
            cache.reserve(c.slot, len(c.tokens))
        for b, c in enumerate(batch.chunks):
            start = cache.length[c.slot]
            n = len(c.tokens)
            base = len(tokens)
            tokens.extend(c.tokens)
            positions.extend(range(start, start + n))
            tok_seq.extend([b] * n)
            cu.append(base + n)
            start_pos.append(start)
            slots.append(c.slot)
            want_rows.extend(base + w for w in c.want)
            max_q = max(max_q, n)
            max_kv = max(max_kv, start + n)
        n_groups = len(cache.groups)
        tables: List[List[int]] = []
        widths: List[int] = []
        for g in range(n_groups):
            width = max(1, max(len(cache.page_lists[s][g]) for s in slots))
            widths.append(width)
            flat: List[int] = []
            for s in slots:
                pl = cache.page_lists[s][g]
                flat.extend(pl)
                flat.extend([-1] * (width - len(pl)))
            tables.append(flat)
        # one host buffer (pinned once and reused; an event says when the last copy out of it is done), one copy
        segments = [tokens, positions, tok_seq, cu, start_pos, slots, want_rows, *tables]
        offsets = []
        total = 0
        for seg_list in segments:
            offsets.append(total)
            total += (len(seg_list) + 3) // 4 * 4                # keep every segment 16-byte aligned
        if getattr(self, "_pinned", None) is None or self._pinned.numel() < total:
            self._pinned = torch.empty(max(total, 4096) * 2, dtype=torch.int32).pin_memory()
            self._pinned_np = self._pinned.numpy()
            self._pinned_event = None
        if self._pinned_event is not None:
            self._pinned_event.synchronize()
        host_np = self._pinned_np
        for off, seg_list in zip(offsets, segments):
            host_np[off:off + len(seg_list)] = seg_list
        dev = torch.empty(total, dtype=torch.int32, device=self.model.runtime.device)
        dev.copy_(self._pinned[:total], non_blocking=True)
        self._pinned_event = torch.cuda.Event()
        self._pinned_event.record()

        def seg(i: int, n: int) -> torch.Tensor:
            return dev[offsets[i]: offsets[i] + n]

        B = len(slots)
        page_tables = [seg(7 + g, B * widths[g]).view(B, widths[g]) for g in range(n_groups)]
        slots_dev = seg(5, B)
        return StepInfo(
            n_tokens=len(tokens), n_seqs=B, max_q_len=max_q, max_kv_len=max_kv,
            tokens=seg(0, len(tokens)), positions=seg(1, len(tokens)), tok_seq=seg(2, len(tokens)),
            cu_seqlens=seg(3, B + 1), start_pos=seg(4, B), slots=slots_dev, want_rows=seg(6, len(want_rows)),
            page_tables=page_tables, slots_long=slots_dev.long(),
        )

    def forward_batch(self, batch: MiniBatch) -> torch.Tensor:
        """Run the batch's tokens; returns float32 logits [number of wanted places, vocab], in
        the order of the batch's sequences and of each one's `want`."""
        batch.validate(self.model.config.vocab_size)
        with torch.cuda.device(self.model.runtime.device):
            step = self.describe(batch)
            logits = self.model.forward(step, self.cache)
            kernels.check_gemm_status(self.model.runtime.device)      # a tensor-core kernel that gave up a wait is an error
        for c in batch.chunks:
            self.cache.commit(c.slot, len(c.tokens))
            self.token_history[c.slot].extend(c.tokens)                      # src/batch.cpp:49
        self.n_steps += 1
        return logits

    # ------------------------------------------------------------------ decoding through a captured graph
    def _runner(self, n_seqs: int, need_len: int, sampler) -> DecodeRunner:
        bucket = 256
        while bucket < need_len:
            bucket *= 2
        bucket = min(bucket, max(need_len, self.max_position))
        p = sampler.params
        key = (n_seqs, bucket, p.greedy) if p.greedy else (n_seqs, bucket, p.temperature, p.top_k, sampler.seed)
        runner = self._runners.get(key)
        if runner is None:
            if len(self._runners) >= 12:
                self._runners.pop(next(iter(self._runners)))
            runner = DecodeRunner(self, n_seqs, bucket, sampler)
            self._runners[key] = runner
        return runner

    def _check_decode(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int) -> None:
        vocab = self.model.config.vocab_size
        if not slots or len(slots) != len(tokens) or len(set(slots)) != len(slots):
            raise ValueError("decode: one token for each of a set of distinct slots")
        for s, t in zip(slots, tokens):
            if s not in self.cache.length:
                raise ValueError(f"decode: slot {s} is not held")
            if not 0 <= int(t) < vocab:
                raise IndexError(f"decode: token id {t} is outside the vocabulary [0, {vocab})")
            if self.cache.length[s] + n_steps > self.max_position:
                raise ContextOverflow(f"slot {s}: {self.cache.length[s]} cached + {n_steps} new tokens pass "
                                      f"max_position_embeddings {self.max_position}")

    def decode_and_sample(self, slots: Sequence[int], tokens: Sequence[int], sampler, seq_ids: Sequence[int]):
        """One decode step for `slots` fed with `tokens`, the next tokens chosen on the device.
        Returns (chosen ids as a list, the step's logits [n, vocab] on the device).  Copies the
        step's inputs to the device and the chosen ids back; `last_copy_bytes` says how much."""
        self._check_decode(slots, tokens, 1)
        slots = list(slots)
        cache = self.cache
        dev = self.model.runtime.device
        if torch.cuda.current_device() != (dev.index or 0):
            torch.cuda.set_device(dev)
        for s in slots:
            cache.reserve(s, 1)
        lengths = [cache.length[s] for s in slots]
        runner = self._runner(len(slots), max(lengths) + 1, sampler)
        h2d = 0
        if runner.graph is None:
            runner.load(slots, tokens, seq_ids)
            runner.capture()
            runner.loaded_slots = None
        if runner.loaded_slots != slots or runner.loaded_ids != list(seq_ids):
            runner.load(slots, tokens, seq_ids)
            runner.loaded_ids = list(seq_ids)
            h2d += runner.host_buf.numel() * 4
        else:
            h2d += runner.load_step(tokens, lengths)
            h2d += runner.refresh_pages(slots)
        runner.replay()
        chosen = runner.read_chosen()
        history = self.token_history
        for s, t in zip(slots, tokens):
            cache.commit(s, 1)
            history[s].append(int(t))
        self.n_steps += 1
        self.last_copy_bytes = (h2d, 4 * len(slots))
        return chosen, runner.logits

    def decode_on_device(self, slots: Sequence[int], tokens: Sequence[int], sampler, seq_ids: Sequence[int],
                         n_steps: int, before=None, after=None) -> torch.Tensor:
        """`n_steps` decode steps back to back without the host in between: every step's chosen
        tokens are the next step's input.  Returns the chosen ids [n_steps, n] (device).
        `before` and `after`, if given, are called around the replays (for timing)."""
        self._check_decode(slots, tokens, n_steps)
        slots = list(slots)
        if n_steps > DecodeRunner.HISTORY_STEPS:
            raise ValueError(f"decode_on_device keeps at most {DecodeRunner.HISTORY_STEPS} steps")
        with torch.cuda.device(self.model.runtime.device):
            for s in slots:
                self.cache.reserve(s, n_steps)
            runner = self._runner(len(slots), max(self.cache.length[s] for s in slots) + n_steps, sampler)
            if runner.graph is None:
                runner.load(slots, tokens, seq_ids)
                runner.capture()
            runner.load(slots, tokens, seq_ids)
            runner.loaded_slots = None                 # the buffers will not describe a host-known state afterwards
            if before is not None:
                before()
            for _ in range(n_steps):
                runner.replay()
            if after is not None:
                after()
            out = runner.history[:n_steps].clone()
        for s in slots:
            self.cache.commit(s, n_steps)
        self.n_steps += n_steps
        return out
