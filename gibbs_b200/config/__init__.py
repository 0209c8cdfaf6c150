from .plan import ModelPlan, LayerSpec, OrderEntry, PartSpec, prenorm_layer
from .registry import register_architecture, known_architectures, detect, parse_config
from .lfm2 import Lfm2Config, ConfigError
from .potivik import PotivikConfig
from .petelix import PetelixConfig
from .sisadra import SisadraConfig
from .selivik import SelivikConfig

register_architecture("Lfm2ForCausalLM", Lfm2Config.from_dict, model_types=("lfm2",))
register_architecture("Potivik", PotivikConfig.from_dict, model_types=("potivik",))
register_architecture("Petelix", PetelixConfig.from_dict, model_types=("petelix",))
register_architecture("Sisadra", SisadraConfig.from_dict, model_types=("sisadra",))
register_architecture("Selivik", SelivikConfig.from_dict, model_types=("selivik",))

__all__ = ["ModelPlan", "LayerSpec", "OrderEntry", "PartSpec", "prenorm_layer", "register_architecture", "known_architectures",
           "detect", "parse_config", "Lfm2Config", "PotivikConfig", "PetelixConfig", "SisadraConfig", "SelivikConfig",
           "ConfigError"]
