"""Decoding as a replayed CUDA graph: one token for each of a fixed set of sequences.

A decode step launches a few kernels per layer, each lasting microseconds; issued one by
one from the host the launches cost more than the kernels.  The runner captures one step
(the model's forward over one token per sequence, the choice of the next token, and a
small kernel that makes the chosen tokens the next step's input and moves every sequence
one position on) into a CUDA graph over fixed buffers.  A step is then: copy the step's
inputs into the buffers (or leave what the previous step put there), replay, read the
chosen tokens.  The captured function is the same `Model.forward` that every other step
runs.

The reference launches its kernels one by one on the default stream and synchronises
after each attention kernel (src/cuda_attention.cu:29-32).
"""
from __future__ import annotations

import contextlib
import gc
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..sampling.sampler import DeviceSampler
from .step_info import StepInfo


def _round_up_pow2(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


@contextlib.contextmanager
def capturing(graph: "torch.cuda.CUDAGraph", stream: "torch.cuda.Stream"):
    """`torch.cuda.graph` with Python's cyclic garbage collector held off: a collection that ran in the middle of a
    capture could free a graph of an earlier context or runner, and destroying a graph while this thread captures
    invalidates the capture."""
    was_on = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        with torch.cuda.graph(graph, stream=stream):
            yield
    finally:
        if was_on:
            gc.enable()


BATCH_SIZES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def padded_batch(n: int) -> int:
    """The batch size a captured step is made for when `n` sequences decode: a batch that shrinks one sequence at a
    time then goes through a dozen captured graphs, not one per size."""
    for b in BATCH_SIZES:
        if n <= b:
            return b
    return (n + 63) // 64 * 64


class DecodeRunner:
    """Buffers and graph for `n_seqs` rows decoding together, valid while no sequence grows beyond `max_len` tokens.
    A batch of fewer sequences fills the remaining rows with copies of its last one: a copy computes the same
    values from the same inputs and writes the same keys and values to the same places, so it changes no result; its
    chosen token is dropped.  (A mixer that keeps state could not tell a copy from a second step, so models with
    state get a runner of the batch's exact size.)  The sampler's seed stands in the buffer, not in the graph."""

    HISTORY_STEPS = 1024

    def __init__(self, context, n_seqs: int, max_len: int, sampler: DeviceSampler):
        self.ctx = context
        self.model = context.model
        self.cache = context.cache
        self.B = n_seqs
        self.max_len = max_len
        self.sampler = sampler
        rt = self.model.runtime
        dev = rt.device
        B = n_seqs
        self.pages_per_seq = max(1, (max_len + self.cache.page_size - 1) // self.cache.page_size)
        n_groups = len(self.cache.groups)
        # one int32 buffer; the per-step inputs come first so that one copy brings them
        names = [("tokens", B), ("positions", B), ("start_pos", B), ("sample_pos", B),
                 ("tok_seq", B), ("cu_seqlens", B + 1), ("slots", B), ("want_rows", B), ("seq_ids", B), ("chosen", B),
                 ("counter", 1), ("seed", 2)] + [(f"pages{g}", B * self.pages_per_seq) for g in range(n_groups)]
        self.offsets = {}
        total = 0
        for name, n in names:
            self.offsets[name] = (total, n)
            total += (n + 3) // 4 * 4
        self.dev_buf = torch.zeros(total, dtype=torch.int32, device=dev)
        self.host_buf = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host_buf.numpy()                       # the same pinned memory, for cheap writes from lists
        self.step_inputs = 4 * B                                    # ints copied to the device at every step
        self.history = torch.zeros(self.HISTORY_STEPS, B, dtype=torch.int32, device=dev)
        self.chosen_host = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.slots_long = torch.zeros(B, dtype=torch.int64, device=dev)
        h = self.host_view
        h("tok_seq")[:] = torch.arange(B, dtype=torch.int32)
        h("cu_seqlens")[:] = torch.arange(B + 1, dtype=torch.int32)
        h("want_rows")[:] = torch.arange(B, dtype=torch.int32)
        for g in range(n_groups):
            h(f"pages{g}")[:] = -1
        self.chosen_dev = self.view("chosen")
        self.chosen_np = self.chosen_host.numpy()
        # the per-step inputs as views made once: slicing a tensor costs microseconds that every step would pay
        end = self.offsets["sample_pos"][0] + B                     # tokens, positions, start_pos, sample_pos lie first
        self._copy_step_in = kernels.PinnedCopy(self.dev_buf[:end], self.host_buf[:end])
        self._copy_chosen_out = kernels.PinnedCopy(self.chosen_host, self.chosen_dev)
        self._np_step = {n: self.host_np[self.offsets[n][0]:self.offsets[n][0] + B]
                         for n in ("tokens", "positions", "start_pos", "sample_pos")}
        self.sync_stream = torch.cuda.current_stream(dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches_per_step = 0
        self.loaded_slots: Optional[List[int]] = None
        self.loaded_ids: Optional[List[int]] = None
        self.loaded_seed: Optional[int] = None
        self.n_live = n_seqs                                        # rows that are sequences of their own, not copies
        self.page_versions: Optional[List[int]] = None            # `SlotBook.page_version` of each slot when its pages were copied

    # ------------------------------------------------------------------ buffers
    def view(self, name: str) -> torch.Tensor:
        o, n = self.offsets[name]
        return self.dev_buf[o:o + n]

    def host_view(self, name: str) -> torch.Tensor:
        o, n = self.offsets[name]
        return self.host_buf[o:o + n]

    def step_info(self) -> StepInfo:
        B = self.B
        tables = [self.view(f"pages{g}").view(B, self.pages_per_seq) for g in range(len(self.cache.groups))]
        return StepInfo(n_tokens=B, n_seqs=B, max_q_len=1, max_kv_len=self.max_len,
                        tokens=self.view("tokens"), positions=self.view("positions"), tok_seq=self.view("tok_seq"),
                        cu_seqlens=self.view("cu_seqlens"), start_pos=self.view("start_pos"), slots=self.view("slots"),
                        want_rows=self.view("want_rows"), page_tables=tables, slots_long=self.slots_long)

    # ------------------------------------------------------------------ one step's body
    def _body(self) -> None:
        step = self.step_info()
        self.logits = self.model.forward(step, self.cache)
        self.sampler.sample_device(self.logits, self.view("seq_ids"), self.view("sample_pos"), out=self.view("chosen"),
                                   seed_on_device=self.view("seed"))
        kernels.decode_advance(self.view("chosen"), self.view("tokens"), self.view("positions"), self.view("start_pos"),
                               self.view("sample_pos"), self.history, self.view("counter"))

    def capture(self) -> None:
        """Run the step once eagerly (libraries initialise, tables are built), then capture it.
        Both runs happen on the buffers' current contents, which must describe valid sequences;
        the caller reloads the buffers afterwards.  The eager run writes the step's keys and values (the
        replay writes the same ones again) and leaves the sequences' fixed-size state as it found it."""
        dev = self.model.runtime.device
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream):
            saved = self.cache.snapshot_state(self.slots_long)      # the warm-up run must not count as a step
            self._body()
            self.cache.restore_state(saved, self.slots_long)
        torch.cuda.current_stream(dev).wait_stream(stream)
        torch.cuda.synchronize(dev)
        before, lib_before = kernels.launch_count(), kernels.library_launch_count()
        self.graph = torch.cuda.CUDAGraph()
        with capturing(self.graph, stream):
            self._body()
        self.launches_per_step = kernels.launch_count() - before
        self.library_launches_per_step = kernels.library_launch_count() - lib_before
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ loading a batch
    def load(self, slots: Sequence[int], tokens: Sequence[int], seq_ids: Sequence[int], seed: Optional[int] = None) -> None:
        """Everything about the batch: called when the set of sequences (or the seed) changes.  Fewer sequences than
        rows: the last one is repeated."""
        B = self.B
        self.n_live = len(slots)
        assert 0 < self.n_live <= B
        pad = B - self.n_live
        slots, tokens, seq_ids = (list(v) + [v[-1]] * pad for v in (slots, tokens, seq_ids))
        seed = self.sampler.seed if seed is None else seed
        h = self.host_view
        h("seed")[0] = (seed & 0xFFFFFFFF) - (1 << 32 if seed & 0x80000000 else 0)
        h("seed")[1] = ((seed >> 32) & 0xFFFFFFFF) - (1 << 32 if (seed >> 32) & 0x80000000 else 0)
        self.loaded_seed = seed
        lengths = [self.cache.length[s] for s in slots]
        h("tokens")[:] = torch.tensor(list(tokens), dtype=torch.int32)
        h("positions")[:] = torch.tensor(lengths, dtype=torch.int32)
        h("start_pos")[:] = h("positions")
        h("sample_pos")[:] = h("positions") + 1
        h("slots")[:] = torch.tensor(list(slots), dtype=torch.int32)
        h("seq_ids")[:] = torch.tensor(list(seq_ids), dtype=torch.int32)
        h("counter")[:] = 0
        self._fill_pages(slots)
        self.dev_buf.copy_(self.host_buf, non_blocking=True)
        if self.cache.has_state:
            self.slots_long.copy_(h("slots").long(), non_blocking=True)
        self.loaded_slots = list(slots[:self.n_live])
        self.loaded_ids = list(seq_ids[:self.n_live])
        self._padded_slots = list(slots)

    def _fill_pages(self, slots: Sequence[int]) -> None:
        P = self.pages_per_seq
        for g in range(len(self.cache.groups)):
            t = self.host_view(f"pages{g}").view(self.B, P)
            for b, s in enumerate(slots):
                pl = self.cache.page_lists[s][g]
                if len(pl) > P:
                    raise RuntimeError("decode runner: a sequence outgrew the runner's page table")
                t[b, :len(pl)] = torch.tensor(pl, dtype=torch.int32)
                t[b, len(pl):] = -1
        self.page_versions = [self.cache.page_version[s] for s in slots]

    def refresh_pages(self, slots: Sequence[int]) -> int:
        """Copy the page tables again if any sequence's pages are not the ones copied last (it got or lost a page, or
        its slot was given back and taken again by another sequence); returns bytes copied."""
        version = self.cache.page_version
        slots = self._padded_slots
        if self.page_versions == [version[s] for s in slots]:
            return 0
        self._fill_pages(slots)
        n = 0
        for g in range(len(self.cache.groups)):
            o, cnt = self.offsets[f"pages{g}"]
            self.dev_buf[o:o + cnt].copy_(self.host_buf[o:o + cnt], non_blocking=True)
            n += cnt * 4
        return n

    def load_step(self, tokens: Sequence[int], lengths: Sequence[int]) -> int:
        """The per-step inputs from the host: tokens and positions.  Returns bytes copied."""
        B = self.B
        pad = B - self.n_live
        if pad:
            tokens, lengths = list(tokens) + [tokens[-1]] * pad, list(lengths) + [lengths[-1]] * pad
        v = self._np_step
        v["tokens"][:] = tokens
        v["positions"][:] = lengths
        np.copyto(v["start_pos"], v["positions"])
        np.add(v["positions"], 1, out=v["sample_pos"])
        self._copy_step_in()
        return self._copy_step_in.nbytes

    def replay(self) -> None:
        self.graph.replay()
        kernels.bindings.count_launches(self.launches_per_step)
        kernels.count_library_launches(self.library_launches_per_step)

    def read_chosen(self) -> List[int]:
        self._copy_chosen_out()
        self.sync_stream.synchronize()
        self.reads = getattr(self, "reads", 0) + 1
        if self.reads % 64 == 1:
            kernels.check_gemm_status(self.model.runtime.device)
        return self.chosen_np[:self.n_live].tolist()
