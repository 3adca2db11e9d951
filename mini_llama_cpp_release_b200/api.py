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
from .engine.engine_config import EngineConfig, parse_dtype  # noqa: F401
from .engine.generate import GenerationResult, generate
from .engine.model import Model
from .sampling.sampler import DeviceSampler, SamplingParams

class LLM:
    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 max_batch_tokens: int = EngineConfig.max_batch_tokens):
        self.model = model
        self.config = model.config
        self.context = Context(model, max_tokens, max_seqs, max_batch_tokens=max_batch_tokens)

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
         max_seqs: Optional[int] = None, max_batch_tokens: Optional[int] = None, engine: Optional[EngineConfig] = None,
         config_path: Optional[str] = None) -> LLM:
    """A model folder (config.json + model.safetensors) → an `LLM` on a CUDA device.  How it runs is an `EngineConfig`,
    given whole as `engine` or by its fields as keywords: `max_tokens` sizes the cache (the most tokens live sequences
    hold at any time, each rounded up to 64), `max_seqs` the number of slots, `max_batch_tokens` the largest step.
    `folder` may also be the path of one .safetensors file; its config.json is then `config_path`, or lies beside it."""
    if engine is None:
        engine = EngineConfig(dtype=dtype, device=device, max_tokens=max_tokens, max_seqs=max_seqs,
                              **({} if max_batch_tokens is None else {"max_batch_tokens": max_batch_tokens}))
    # float32 products must be float32: no TF32, no reduced-precision accumulation
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model = Model.from_folder(folder, engine.dtype, engine.device, config_path=config_path)
    llm = LLM(model, engine.max_tokens, engine.max_seqs, engine.max_batch_tokens)
    llm.engine = engine
    return llm
