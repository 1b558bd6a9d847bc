"""Configuration: typed specs, the Qwen3 reader and the architecture registry."""
from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE, Qwen3Config
from .registry import (model_spec_from_dict, model_spec_from_folder, read_config_json,
                       read_generation_stop_ids,
                       register_architecture, registered_architectures)

register_architecture(QWEN3_ARCHITECTURE, lambda d: Qwen3Config.from_dict(d).to_model_spec(d))

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config",
           "QWEN3_ARCHITECTURE", "model_spec_from_dict", "model_spec_from_folder",
           "read_config_json", "read_generation_stop_ids", "register_architecture", "registered_architectures"]
