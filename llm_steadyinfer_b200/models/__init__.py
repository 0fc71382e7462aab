from . import llama, mivorax, nufasun, vibunex  # noqa: F401  (register "LlamaForCausalLM", "Mivorax", "Nufasun", "Vibunex")
from .model import Model
