from .spec import PartSpec, LayerSpec, ScheduleEntry, ModelSpec
from .dense import DenseDecoderConfig, RopeScaling
from .registry import ARCHITECTURES, register_architecture, describe, read_config_json
from .engine_config import EngineConfig

__all__ = ["PartSpec", "LayerSpec", "ScheduleEntry", "ModelSpec", "DenseDecoderConfig", "RopeScaling",
           "ARCHITECTURES", "register_architecture", "describe", "read_config_json", "EngineConfig"]
