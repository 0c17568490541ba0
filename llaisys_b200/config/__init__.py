from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec
from .registry import config_from_dict, known_architectures, load_config, register_architecture
from .qwen2 import Qwen2Config
from .vumezen import VumezenConfig
from .nubedra import NubedraConfig
from .zedirax import ZediraxConfig
from .zetalorn import ZetalornConfig

__all__ = ["CallSpec", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "SubLayerSpec", "Qwen2Config", "VumezenConfig", "NubedraConfig", "ZediraxConfig", "ZetalornConfig",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]
