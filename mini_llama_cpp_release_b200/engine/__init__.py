from .batch import MiniBatch, SequenceChunk  # noqa: F401
from .step_info import StepInfo  # noqa: F401
from .model import Model, build_parts  # noqa: F401
from .context import Context, ContextOverflow  # noqa: F401
from .generate import GenerationResult, generate, plan_batches, check_request_sizes  # noqa: F401
from .engine_config import EngineConfig, parse_dtype  # noqa: F401
