"""What a step looks like to the parts: the tokens of all sequences packed back to back,
and, for every token and every sequence, where it is.

All index tensors are int32 on the device.  Host-side integers (`n_tokens`, `n_seqs`,
`max_q_len`, `max_kv_len`) size grids and scratch memory; kernels take each sequence's
true lengths from the device tensors, so a bound that is larger than needed changes no
result.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class StepInfo:
    n_tokens: int                 # tokens of this step, over all sequences
    n_seqs: int
    max_q_len: int                # longest run of new tokens of any sequence
    max_kv_len: int               # longest sequence after this step
    tokens: torch.Tensor          # [n_tokens] token ids
    positions: torch.Tensor       # [n_tokens] position of each token in its sequence
    tok_seq: torch.Tensor         # [n_tokens] index (in this step) of each token's sequence
    cu_seqlens: torch.Tensor      # [n_seqs + 1] first token of each sequence in the packed order
    start_pos: torch.Tensor       # [n_seqs] tokens each sequence had before this step
    slots: torch.Tensor           # [n_seqs] cache slot of each sequence
    want_rows: torch.Tensor       # [n_want] packed token rows whose logits are asked for
    page_tables: List[torch.Tensor]   # per cache group: [n_seqs, pages] page of each page index, -1: none
    slots_long: Optional[torch.Tensor] = None   # [n_seqs] int64 copy of `slots`, for indexing state tensors; None when no mixer of the model declared state

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1
