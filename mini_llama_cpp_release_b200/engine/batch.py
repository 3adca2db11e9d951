"""The unit of work of the step function: for each sequence of the batch, its next tokens.

The reference's `MiniBatch` is the tokens and positions of one sequence, and its
`forward_batch` walks them one by one and returns the last token's logits
(include/mini_llama/batch.h:9-23; src/batch.cpp:33-52).  Here a batch holds several
sequences, each bound to a cache slot, each continuing at the slot's current length; the
positions follow from that and are not given twice.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


@dataclass
class SequenceChunk:
    slot: int
    tokens: List[int]
    want: List[int] = field(default_factory=list)      # indices into `tokens` whose logits are asked for


@dataclass
class MiniBatch:
    chunks: List[SequenceChunk]

    @property
    def n_tokens(self) -> int:
        return sum(len(c.tokens) for c in self.chunks)

    @staticmethod
    def single(slot: int, token: int, want: bool = True) -> "MiniBatch":
        """One token of one sequence (include/mini_llama/batch.h:18-19)."""
        return MiniBatch([SequenceChunk(slot, [int(token)], [0] if want else [])])

    @staticmethod
    def from_tokens(slot: int, tokens: Sequence[int], want: Optional[Sequence[int]] = None) -> "MiniBatch":
        """Several tokens of one sequence, continuing where the slot stands
        (include/mini_llama/batch.h:21-23); by default the last token's logits are wanted."""
        toks = [int(t) for t in tokens]
        return MiniBatch([SequenceChunk(slot, toks, list(want) if want is not None else [len(toks) - 1])])

    @staticmethod
    def prefill(slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> "MiniBatch":
        """Whole prompts of several sequences in one step; each one's last position is wanted."""
        if len(slots) != len(prompts):
            raise ValueError("one slot per prompt")
        return MiniBatch([SequenceChunk(s, [int(t) for t in p], [len(p) - 1]) for s, p in zip(slots, prompts)])

    @staticmethod
    def decode(slots: Sequence[int], tokens: Sequence[int]) -> "MiniBatch":
        """One token for each of several sequences."""
        if len(slots) != len(tokens):
            raise ValueError("one token per slot")
        return MiniBatch([SequenceChunk(s, [int(t)], [0]) for s, t in zip(slots, tokens)])

    def validate(self, vocab_size: int) -> None:
        """Empty batches, empty sequences, a slot named twice, token ids outside the
        vocabulary and wanted places outside a sequence are errors
        (src/batch.cpp:38-43; src/forward.cpp:20-22)."""
        if not self.chunks:
            raise ValueError("forward_batch: the batch is empty")
        seen = set()
        for c in self.chunks:
            if not c.tokens:
                raise ValueError(f"forward_batch: slot {c.slot} brings no tokens")
            if c.slot in seen:
                raise ValueError(f"forward_batch: slot {c.slot} appears twice in one batch")
            seen.add(c.slot)
            for t in c.tokens:
                if not 0 <= t < vocab_size:
                    raise IndexError(f"forward_batch: token id {t} is outside the vocabulary [0, {vocab_size})")
            for w in c.want:
                if not 0 <= w < len(c.tokens):
                    raise IndexError(f"forward_batch: wanted place {w} is outside the {len(c.tokens)} tokens of slot {c.slot}")

    def split(self, max_tokens: int) -> List[Tuple["MiniBatch", List[Tuple[int, int]]]]:
        """The batch cut into steps of at most `max_tokens` tokens, sequence by sequence in order: a step takes whole
        sequences while they fit and then the first part of the next one, whose rest opens the following step (it
        continues where the cache then stands, so nothing but the cut differs).  With each step comes, for every
        row of logits it will return, which wanted place of the original batch it is: (index of the sequence,
        index into that sequence's `want`)."""
        if max_tokens < 1:
            raise ValueError("a step must be allowed at least one token")
        pieces: List[Tuple[MiniBatch, List[Tuple[int, int]]]] = []
        cur: List[SequenceChunk] = []
        keys: List[Tuple[int, int]] = []
        room = max_tokens
        for e, c in enumerate(self.chunks):
            lo = 0
            while lo < len(c.tokens):
                take = min(room, len(c.tokens) - lo)
                here = [(j, w - lo) for j, w in enumerate(c.want) if lo <= w < lo + take]
                cur.append(SequenceChunk(c.slot, c.tokens[lo:lo + take], [w for _, w in here]))
                keys.extend((e, j) for j, _ in here)
                lo += take
                room -= take
                if room == 0:
                    pieces.append((MiniBatch(cur), keys))
                    cur, keys, room = [], [], max_tokens
        if cur:
            pieces.append((MiniBatch(cur), keys))
        return pieces
