from .schema import Qwen3Config, GenerationDefaults, read_json, FULL_ATTENTION, SLIDING_ATTENTION
from .registry import (Architecture, register_architecture, resolve_architecture, load_config,
                       architecture_names)
from .surelorn import SurelornConfig
from .bumisun import BumisunConfig
from .pamarax import PamaraxConfig
from .tebozen import TebozenConfig
