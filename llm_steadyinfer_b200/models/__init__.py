from . import llama, mivorax  # noqa: F401  (register "LlamaForCausalLM", "Mivorax")
from .model import Model
