from . import qwen3  # registers Qwen3ForCausalLM
from . import surelorn  # registers Surelorn
from . import bumisun  # registers Bumisun
from . import pamarax  # registers Pamarax
from . import tebozen  # registers Tebozen
