"""A context: one model's cache on one device, and the step function over it.

The reference's context is one sequence: its cache, its position, its token history
(include/mini_llama/context.h:11-30), and `forward_batch(model, ctx, batch)` feeds it
(src/batch.cpp:33-52).  Here a context holds many sequences, each in a slot; a step
brings the next tokens of some of them, runs exactly those tokens as one batch against
the cache, and returns logits at the places asked for.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.paged import PAGE_SIZE, PagedCache
from .batch import MiniBatch, SequenceChunk
from .decode_runner import DecodeRunner, capturing, padded_batch
from .model import Model
from .step_info import StepInfo


class ContextOverflow(ValueError):
    """A sequence would pass the model's largest position."""


class Context:
    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None, page_size: int = PAGE_SIZE,
                 max_batch_tokens: int = 16384):
        """`max_tokens`: the most tokens live sequences hold at any time, each sequence's
        count rounded up to whole pages of `page_size` tokens.  `max_batch_tokens`: the most
        tokens one step runs at once; a larger batch is run as several steps."""
        self.model = model
        if max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be positive")
        self.max_batch_tokens = int(max_batch_tokens)
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
    def _describe_host(self, batch: MiniBatch) -> dict:
        """Reserve pages for the batch's tokens and write the step's description into the pinned host buffer; returns
        its layout (segment offsets and the sizes the host needs)."""
        cache = self.cache
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
        B = len(batch.chunks)
        slots = [c.slot for c in batch.chunks]
        lens = [len(c.tokens) for c in batch.chunks]
        start_pos = [cache.length[s] for s in slots]
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        n_tokens = cu[-1]
        want_rows = [cu[b] + w for b, c in enumerate(batch.chunks) for w in c.want]
        max_q = max(lens)
        max_kv = max(s + n for s, n in zip(start_pos, lens))
        n_groups = len(cache.groups)
        widths = [max(1, max(len(cache.page_lists[s][g]) for s in slots)) for g in range(n_groups)]
        # one host buffer (pinned once and reused; an event says when the last copy out of it is done), one copy.
        # Segments: tokens, positions, sequence of each token, first token of each sequence, first position of each
        # sequence, slots, wanted rows, then one page table per cache group; each 16-byte aligned.
        sizes = [n_tokens, n_tokens, n_tokens, B + 1, B, B, len(want_rows)] + [B * w for w in widths]
        offsets = []
        total = 0
        for size in sizes:
            offsets.append(total)
            total += (size + 3) // 4 * 4
        if getattr(self, "_pinned", None) is None or self._pinned.numel() < total:
            self._pinned = torch.empty(max(total, 4096) * 2, dtype=torch.int32).pin_memory()
            self._pinned_np = self._pinned.numpy()
            self._pinned_event = None
        if self._pinned_event is not None:
            self._pinned_event.synchronize()
        host_np = self._pinned_np
        # the per-token segments are filled a sequence at a time, as arrays: a prompt of thousands of tokens is not
        # walked in Python
        for b, c in enumerate(batch.chunks):
            lo, n = cu[b], lens[b]
            host_np[offsets[0] + lo: offsets[0] + lo + n] = c.tokens
            host_np[offsets[1] + lo: offsets[1] + lo + n] = np.arange(start_pos[b], start_pos[b] + n, dtype=np.int32)
            host_np[offsets[2] + lo: offsets[2] + lo + n] = b
        host_np[offsets[3]: offsets[3] + B + 1] = cu
        host_np[offsets[4]: offsets[4] + B] = start_pos
        host_np[offsets[5]: offsets[5] + B] = slots
        host_np[offsets[6]: offsets[6] + len(want_rows)] = want_rows
        for g in range(n_groups):
            w = widths[g]
            table = host_np[offsets[7 + g]: offsets[7 + g] + B * w].reshape(B, w)
            table[:] = -1
            for b, s in enumerate(slots):
                pl = cache.page_lists[s][g]
                table[b, :len(pl)] = pl
        return dict(total=total, offsets=offsets, n_tokens=n_tokens, n_seqs=B, max_q=max_q, max_kv=max_kv,
                    widths=widths, n_want=len(want_rows))

    def _upload(self, layout: dict, into: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The description `_describe_host` left in the pinned buffer, copied to the device (into `into` if given)."""
        total = layout["total"]
        if into is None:
            into = torch.empty(total, dtype=torch.int32, device=self.model.runtime.device)
        into.copy_(self._pinned[:total], non_blocking=True)
        self._pinned_event = torch.cuda.Event()
        self._pinned_event.record()
        return into

    def describe(self, batch: MiniBatch) -> StepInfo:
        """Reserve pages for the batch's tokens and put its description on the device."""
        layout = self._describe_host(batch)
        return self._step_over(self._upload(layout), layout)

    @staticmethod
    def _step_key(layout: dict) -> tuple:
        """Everything about a step that the host bakes into launches (grids, strides, the kernels chosen); whatever else
        differs between two steps lies in the description on the device."""
        return (layout["n_tokens"], layout["n_seqs"], layout["max_q"], layout["max_kv"], tuple(layout["widths"]),
                layout["n_want"])

    def _step_over(self, dev: torch.Tensor, layout: dict) -> StepInfo:
        """The step's description as views of `dev`, the int32 buffer `describe` filled."""
        offsets, B, n_tokens, widths = layout["offsets"], layout["n_seqs"], layout["n_tokens"], layout["widths"]

        def seg(i: int, n: int) -> torch.Tensor:
            return dev[offsets[i]: offsets[i] + n]

        page_tables = [seg(7 + g, B * widths[g]).view(B, widths[g]) for g in range(len(widths))]
        slots_dev = seg(5, B)
        return StepInfo(
            n_tokens=n_tokens, n_seqs=B, max_q_len=layout["max_q"], max_kv_len=layout["max_kv"],
            tokens=seg(0, n_tokens), positions=seg(1, n_tokens), tok_seq=seg(2, n_tokens),
            cu_seqlens=seg(3, B + 1), start_pos=seg(4, B), slots=slots_dev, want_rows=seg(6, layout["n_want"]),
            page_tables=page_tables, slots_long=slots_dev.long() if self.cache.has_state else None,
        )

    # A step of many tokens is some two hundred launches issued from Python; when its kernels are fast the host
    # becomes the limit.  A shape of step that comes again (the same numbers of tokens and sequences, the same
    # longest lengths: fixed-size prompts, a benchmark, chunks of a fixed size) is therefore captured into a CUDA
    # graph the second time it is seen and replayed from then on; everything that may differ between two such
    # steps (tokens, positions, lengths, pages) lies in the description buffer the graph reads.
    STEP_GRAPHS = 4                     # captured shapes kept
    STEP_GRAPH_MIN_TOKENS = 64          # smaller steps are cheap to issue

    def forward_batch(self, batch: MiniBatch) -> torch.Tensor:
        """Run the batch's tokens; returns float32 logits [number of wanted places, vocab], in
        the order of the batch's sequences and of each one's `want`.  A batch of more than
        `max_batch_tokens` tokens runs as several steps, cut sequence by sequence; the later
        part of a cut sequence continues from the cache like any later chunk of it would."""
        batch.validate(self.model.config.vocab_size)
        if batch.n_tokens <= self.max_batch_tokens:
            return self._forward_step(batch)
        # everything that can be refused is refused before the first piece runs
        for c in batch.chunks:
            if c.slot not in self.cache.length:
                raise ValueError(f"forward_batch: slot {c.slot} is not held")
            if self.cache.length[c.slot] + len(c.tokens) > self.max_position:
                raise ContextOverflow(f"slot {c.slot}: {self.cache.length[c.slot]} cached + {len(c.tokens)} new tokens pass "
                                      f"max_position_embeddings {self.max_position}")
        self.cache.reserve_all([(c.slot, len(c.tokens)) for c in batch.chunks])
        outs, keys = [], []
        for piece, piece_keys in batch.split(self.max_batch_tokens):
            outs.append(self._forward_step(piece))
            keys.extend(piece_keys)
        self.n_steps -= len(outs) - 1                      # one call, one step in the count
        wanted = [(e, j) for e, c in enumerate(batch.chunks) for j in range(len(c.want))]
        logits = torch.cat(outs, dim=0)
        if keys == wanted:
            return logits
        row_of = {k: r for r, k in enumerate(keys)}
        order = torch.tensor([row_of[k] for k in wanted], dtype=torch.long, device=logits.device)
        return logits.index_select(0, order)

    def _forward_step(self, batch: MiniBatch) -> torch.Tensor:
        """One step: all of the batch's tokens at once."""
        dev = self.model.runtime.device
        with torch.cuda.device(dev):
            n_new = sum(len(c.tokens) for c in batch.chunks)
            if self.use_graphs and n_new >= self.STEP_GRAPH_MIN_TOKENS:
                logits = self._forward_maybe_replayed(batch)
            else:
                step = self.describe(batch)
                logits = self.model.forward(step, self.cache)
            kernels.check_gemm_status(dev)      # a tensor-core kernel that gave up a wait is an error
        for c in batch.chunks:
            self.cache.commit(c.slot, len(c.tokens))
            self.token_history[c.slot].extend(c.tokens)                      # src/batch.cpp:49
        self.n_steps += 1
        return logits

    def _forward_maybe_replayed(self, batch: MiniBatch) -> torch.Tensor:
        graphs = self.__dict__.setdefault("_step_graphs", {})
        seen = self.__dict__.setdefault("_step_shapes_seen", {})
        dev = self.model.runtime.device
        layout = self._describe_host(batch)
        key = self._step_key(layout)
        entry = graphs.get(key)
        if entry is not None:
            self._upload(layout, into=entry["dev"])
            entry["graph"].replay()
            graphs[key] = graphs.pop(key)                                     # most recently used last
            return entry["logits"].clone()
        seen[key] = seen.get(key, 0) + 1
        if len(seen) > 64:
            seen.pop(next(iter(seen)))
        own = self._upload(layout)
        if seen[key] < 2:
            return self.model.forward(self._step_over(own, layout), self.cache)
        # second time: run it once more eagerly on a side stream (what capture needs), then capture and replay
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream):
            warm = self._step_over(own, layout)
            saved = self.cache.snapshot_state(warm.slots_long)      # the warm-up run must not count as a step
            self.model.forward(warm, self.cache)
            self.cache.restore_state(saved, warm.slots_long)
        torch.cuda.current_stream(dev).wait_stream(stream)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with capturing(graph, stream):
            logits = self.model.forward(self._step_over(own, layout), self.cache)
        torch.cuda.synchronize(dev)
        while len(graphs) >= self.STEP_GRAPHS:
            graphs.pop(next(iter(graphs)))
        graphs[key] = dict(graph=graph, dev=own, logits=logits)
        graph.replay()
        return logits.clone()

    # ------------------------------------------------------------------ decoding through a captured graph
    def _runner(self, n_seqs: int, need_len: int, sampler) -> DecodeRunner:
        bucket = 256
        while bucket < need_len:
            bucket *= 2
        bucket = min(bucket, max(need_len, self.max_position))
        p = sampler.params
        # the rows of the captured step: the batch's size rounded up to one of a few (the spare rows repeat a sequence,
        # which is only sound while no mixer keeps state of its own); the seed is data in the runner's buffer
        rows = n_seqs if self.cache.has_state else padded_batch(n_seqs)
        key = (rows, bucket, p.greedy) if p.greedy else (rows, bucket, p.temperature, p.top_k)
        runner = self._runners.get(key)
        if runner is None:
            if len(self._runners) >= 24:
                self._runners.pop(next(iter(self._runners)))
            runner = DecodeRunner(self, rows, bucket, sampler)
            self._runners[key] = runner
        else:
            self._runners[key] = self._runners.pop(key)            # most recently used last
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
            runner.load(slots, tokens, seq_ids, sampler.seed)
            runner.capture()
            runner.loaded_slots = None
        if runner.loaded_slots != slots or runner.loaded_ids != list(seq_ids) or runner.loaded_seed != sampler.seed:
            runner.load(slots, tokens, seq_ids, sampler.seed)
            h2d += runner.host_buf.numel() * 4
        else:
            h2d += runner.load_step(tokens, lengths)
            h2d += runner.refresh_pages(slots)
        runner.replay()
        # the host's bookkeeping of this step while the device runs it
        history = self.token_history
        for s, t in zip(slots, tokens):
            cache.commit(s, 1)
            history[s].append(int(t))
        self.n_steps += 1
        chosen = runner.read_chosen()
        logits = runner.logits[:len(slots)]
        self.last_copy_bytes = (h2d, 4 * len(slots))
        return chosen, logits

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
                runner.load(slots, tokens, seq_ids, sampler.seed)
                runner.capture()
            runner.load(slots, tokens, seq_ids, sampler.seed)
            runner.loaded_slots = None                 # the buffers will not describe a host-known state afterwards
            if before is not None:
                before()
            for _ in range(n_steps):
                runner.replay()
            if after is not None:
                after()
            out = runner.history[:n_steps, :len(slots)].clone()
        for s in slots:
            self.cache.commit(s, n_steps)
        self.n_steps += n_steps
        return out
