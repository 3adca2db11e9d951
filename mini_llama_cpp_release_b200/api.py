"""The Python entry point: load a model folder, generate from token ids.

The reference has no Python binding; its one-shot entry is `mini-llama generate`
(src/main.cpp:506-746).  `LLM.generate` takes the same knobs under the same names
(`n_predict`, `temperature`, `top_k`, `seed`) and returns token ids; there is no tokenizer
here, prompts are lists of ids.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from .engine.context import Context
from .engine.generate import GenerationResult, generate
from .engine.model import Model
from .sampling.sampler import DeviceSampler, SamplingParams

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


class LLM:
    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None):
        self.model = model
        self.config = model.config
        self.context = Context(model, max_tokens, max_seqs)

    def generate(self, prompts: Sequence[Sequence[int]], n_predict: Union[int, Sequence[int]] = 16, temperature: float = 0.0,
                 top_k: int = 0, seed: int = 0, stop_token_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None, return_details: bool = False, on_step=None
                 ) -> Union[List[List[int]], List[GenerationResult]]:
        """Generated ids for each prompt (lists of token ids).  `n_predict` is one number for all
        requests or one per request.  `stop_token_ids` defaults to the
        checkpoint's `eos_token_id`, if it has one.  `on_step(live, chosen, logits)`, if given, is
        called after every choice with the indices of the live requests, their chosen ids and
        the logits they were chosen from."""
        if stop_token_ids is None:
            stop_token_ids = self.config.eos_token_id or ()
        sampler = DeviceSampler(SamplingParams(temperature, top_k, seed), self.model.runtime.device)
        results = generate(self.context, sampler, prompts, n_predict, stop_token_ids, max_batch=max_batch,
                           on_step=on_step)
        return results if return_details else [r.tokens for r in results]


def load(folder: str, dtype="bfloat16", device: str = "cuda:0", max_tokens: int = 8192,
         max_seqs: Optional[int] = None) -> LLM:
    """A model folder (config.json + model.safetensors) → an `LLM` on `device`.  `max_tokens`
    sizes the cache: the most tokens live sequences hold at any time, each rounded up to 64."""
    # float32 products must be float32: no TF32, no reduced-precision accumulation
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model = Model.from_folder(folder, parse_dtype(dtype), device)
    return LLM(model, max_tokens, max_seqs)
