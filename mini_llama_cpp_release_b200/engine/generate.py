"""The generation loop above the step function.

For one sequence the contract is the reference's (src/main.cpp:686-709): prefill the
prompt, take the first token from the logits of its last position, then feed each chosen
token back and choose the next; `n_predict` counts the first chosen token; the last chosen
token is never fed; `n_predict == 0` generates nothing.  What is new: several sequences
with unequal prompts start together in one prefill step; `n_predict` may be one number for
all requests or one per request; a sequence that ends (stop token
or `n_predict` reached) leaves the batch while the others go on; when there are more
requests than one batch holds, batches run one after another and reuse the slots and pages
the previous batch gave back.

A stop token is kept in the output and ends its sequence; it is checked after every
choice, the first included (the reference skips the check for the first one,
src/main.cpp:692-693 against 706-708).

The loop only needs `acquire`, `release` and `forward_batch` from its context and
`sample` from its sampler, so its decisions are tested on the CPU with stand-ins.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Set, Union

from .batch import MiniBatch, SequenceChunk


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = "length"          # "stop": a stop token was chosen; "length": n_predict reached
    prompt_len: int = 0


def per_request(n_predict: Union[int, Sequence[int]], n_requests: int) -> List[int]:
    """`n_predict` as a list with one entry per request."""
    if isinstance(n_predict, int):
        return [n_predict] * n_requests
    out = [int(n) for n in n_predict]
    if len(out) != n_requests:
        raise ValueError(f"n_predict has {len(out)} entries for {n_requests} requests")
    return out


def check_request_sizes(prompt_lens: Sequence[int], n_predict: Union[int, Sequence[int]], max_position: int) -> None:
    """Reject up front what cannot fit (src/main.cpp:656-663)."""
    counts = per_request(n_predict, len(prompt_lens))
    if any(n < 0 for n in counts):
        raise ValueError("n_predict must not be negative")
    for i, n in enumerate(prompt_lens):
        n_predict = counts[i]
        if n <= 0:
            raise ValueError(f"request {i}: the prompt is empty")
        if n > max_position:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the model's {max_position} positions")
        # the last chosen token is never fed, so a sequence stores prompt + n_predict - 1 tokens
        if n + max(0, n_predict - 1) > max_position:
            raise ValueError(f"request {i}: prompt of {n} tokens plus {n_predict} to generate exceeds the model's "
                             f"{max_position} positions")


def plan_batches(prompt_lens: Sequence[int], n_predict: Union[int, Sequence[int]], page_size: int, n_pages: int,
                 max_seqs: int, max_batch: Optional[int] = None) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the cache: at most `max_seqs` (and
    `max_batch`) sequences, and pages for every sequence at its final length."""
    limit = max_seqs if max_batch is None else max(1, min(max_seqs, max_batch))
    counts = per_request(n_predict, len(prompt_lens))
    batches: List[List[int]] = []
    cur: List[int] = []
    cur_pages = 0
    for i, n in enumerate(prompt_lens):
        final_len = n + max(0, counts[i] - 1)
        pages = (final_len + page_size - 1) // page_size
        if pages > n_pages:
            raise ValueError(f"request {i} needs {pages} cache pages of {page_size} tokens; the cache has {n_pages}")
        if cur and (len(cur) >= limit or cur_pages + pages > n_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += pages
    if cur:
        batches.append(cur)
    return batches


def generate_batch(ctx, sampler, prompts: Sequence[Sequence[int]], seq_ids: Sequence[int],
                   n_predict: Union[int, Sequence[int]], stop: Set[int], on_step: Optional[Callable] = None
                   ) -> List[GenerationResult]:
    """One batch of sequences that start together.  A request that asks for no tokens takes no slot and runs nothing."""
    results = [GenerationResult(prompt_len=len(p)) for p in prompts]
    counts = per_request(n_predict, len(prompts))
    live = [i for i in range(len(prompts)) if counts[i] > 0]
    if not live:
        return results
    slots = [ctx.acquire() if counts[i] > 0 else -1 for i in range(len(prompts))]
    try:
        lengths = [len(p) for p in prompts]
        logits = ctx.forward_batch(MiniBatch.prefill([slots[i] for i in live], [prompts[i] for i in live]))
        fused = bool(getattr(ctx, "use_graphs", False)) and hasattr(ctx, "decode_and_sample")
        live_slots, live_ids = [slots[i] for i in live], [seq_ids[i] for i in live]
        chosen_next = None
        while True:
            if chosen_next is not None:
                chosen, chosen_next = chosen_next, None
            else:
                chosen = sampler.sample(logits, live_ids, [lengths[i] for i in live])
            if on_step is not None:
                on_step(live, chosen, logits)
            still: List[int] = []
            feed: List[int] = []
            for i, tok in zip(live, chosen):
                tok = int(tok)
                results[i].tokens.append(tok)
                if tok in stop:
                    results[i].finish_reason = "stop"
                elif len(results[i].tokens) >= counts[i]:
                    results[i].finish_reason = "length"
                else:
                    still.append(i)
                    feed.append(tok)
            if len(still) != len(live):
                for i in live:
                    if i not in still:
                        ctx.release(slots[i])      # a finished sequence gives its slot and pages back at once
                        slots[i] = -1
                live = still
                live_slots, live_ids = [slots[i] for i in live], [seq_ids[i] for i in live]
            if not live:
                break
            for i in live:
                lengths[i] += 1
            if fused:
                # forward, choice and the move to the next position are one captured graph
                chosen_next, logits = ctx.decode_and_sample(live_slots, feed, sampler, live_ids)
            else:
                logits = ctx.forward_batch(MiniBatch.decode(live_slots, feed))
    finally:
        for s in slots:
            if s >= 0:
                ctx.release(s)
    return results


def generate(ctx, sampler, prompts: Sequence[Sequence[int]], n_predict: Union[int, Sequence[int]],
             stop_token_ids: Sequence[int] = (),
             max_position: Optional[int] = None, max_batch: Optional[int] = None,
             on_step: Optional[Callable] = None) -> List[GenerationResult]:
    """All requests, in as many batches as the cache needs."""
    prompts = [list(map(int, p)) for p in prompts]
    lens = [len(p) for p in prompts]
    if max_position is None:
        max_position = ctx.max_position
    counts = per_request(n_predict, len(prompts))
    check_request_sizes(lens, counts, max_position)
    book = ctx.cache
    batches = plan_batches(lens, counts, book.page_size, book.n_pages, book.max_seqs, max_batch)
    out: List[Optional[GenerationResult]] = [None] * len(prompts)
    stop = set(int(t) for t in stop_token_ids)
    for ids in batches:
        # the observer hears the requests' indices in this call, not their places in the batch
        hook = None if on_step is None else (lambda live, chosen, logits, ids=ids: on_step([ids[i] for i in live], chosen, logits))
        res = generate_batch(ctx, sampler, [prompts[i] for i in ids], ids, [counts[i] for i in ids], stop, hook)
        for i, r in zip(ids, res):
            out[i] = r
    return out  # type: ignore[return-value]
