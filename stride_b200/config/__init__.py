from .engine import DTYPES, EngineConfig
from .llama import LlamaConfig
from .nidilix import NidilixConfig
from .migelix import MigelixConfig
from .tutizen import TutizenConfig
from .netusun import NetusunConfig
from .memory import B200_MEMORY_BYTES, MemoryPlan, PlanError, plan_memory
from .presets import PRESETS, preset
from .registry import (ConfigError, config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .specs import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PassInputSpec, PositionSpec, RopeScaling, ScheduleEntry,
                    StreamInputSpec, default_schedule)

__all__ = [
    "DTYPES", "EngineConfig", "LlamaConfig", "NidilixConfig", "MigelixConfig", "TutizenConfig", "NetusunConfig", "StreamInputSpec", "MemoryPlan", "PlanError", "plan_memory", "B200_MEMORY_BYTES", "PRESETS", "preset", "ConfigError", "config_class_for", "config_from_dict",
    "load_config", "register_architecture", "registered_architectures", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec", "LayerSpec", "MixerSpec",
    "ModelSpec", "NormSpec", "PassInputSpec", "PositionSpec", "RopeScaling", "ScheduleEntry", "default_schedule",
]
