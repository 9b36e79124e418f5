from . import llama, mivorax, nufasun  # noqa: F401  (register "LlamaForCausalLM", "Mivorax", "Nufasun")
from .model import Model
