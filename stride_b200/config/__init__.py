from .llama import ConfigError, LlamaConfig, RopeScaling
from .registry import Architecture, register_architecture, registered_architectures, resolve_architecture
from . import llama_spec as _llama_spec  # registers LlamaForCausalLM

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "Architecture", "register_architecture",
           "registered_architectures", "resolve_architecture"]
