from .decoder import DecoderModel, LayerCall
from . import qwen3  # registers "Qwen3ForCausalLM"
from . import zidivik  # registers "Zidivik"
from . import tidavik  # registers "Tidavik"
from . import toredra  # registers "Toredra"
from . import korirax  # registers "Korirax"

__all__ = ["DecoderModel", "LayerCall", "qwen3", "zidivik", "tidavik", "toredra", "korirax"]
