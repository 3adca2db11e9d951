"""A small, whole inference library for the Qwen2 dense decoder on one NVIDIA B200.

    import mini_llama_cpp_release_b200 as ml
    llm = ml.load("model_folder", dtype="bfloat16", max_tokens=8192)
    out = llm.generate([[1, 2, 3], [4, 5]], n_predict=16)            # greedy
    out = llm.generate(prompts, n_predict=16, temperature=0.8, top_k=40, seed=7)

`ml.load` gives an `LLM`: a model bound to its weights plus a context (cache and step
function).  `ml.write_random_model(config, folder, seed)` makes a model folder with random
weights.  `python -m mini_llama_cpp_release_b200 generate|bench|inspect|replay` is the
command line; `bin/trace_run` replays token traces.
"""
from .api import LLM, load  # noqa: F401
from .engine.engine_config import EngineConfig  # noqa: F401
from .config import ConfigError, ModelConfig, register_architecture, register_part  # noqa: F401
from .engine import Context, MiniBatch, Model  # noqa: F401
from .sampling import SamplingParams  # noqa: F401
from .weights import WeightError, write_random_model  # noqa: F401

__version__ = "0.1.0"
