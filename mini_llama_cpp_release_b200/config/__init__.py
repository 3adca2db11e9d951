from .model_config import ConfigError, ModelConfig  # noqa: F401
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, prenorm_layer, sequential_schedule  # noqa: F401
from .registry import (build_model_spec, build_part, config_class_of, known_architectures, part_class,  # noqa: F401
                       register_architecture, register_part)
