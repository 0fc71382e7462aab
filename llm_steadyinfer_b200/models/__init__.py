from . import fevosun, llama, mivorax, nufasun, vibunex  # noqa: F401  (register "Fevosun", "LlamaForCausalLM", "Mivorax", "Nufasun", "Vibunex")
from .model import Model
