from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, save_safetensors  # noqa: F401
from .loader import WeightError, compare, expected_tensors, load_weights  # noqa: F401
from .random_init import random_tensor, write_random_model  # noqa: F401
