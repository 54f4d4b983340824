"""synaptix_b200: a small model library with generation of its own for one GPU (sm_100a).

Everything between a request's tokens and its next token for the Qwen3 dense
decoder: typed configuration and registry, weights from safetensors (or seeded
random weights), layers put together from parts, a paged cache with a slot per
sequence, one step function over unequal batches, a generation loop, sampling,
and hand-written CUDA kernels with a true 32-bit path beside the bfloat16 one.
"""
from .config import ConfigError, Qwen3Config, load_config, register_architecture
from .weights import WeightError, write_model_folder
from .api import LLM, generate, load_llm

__version__ = "0.1.0"

__all__ = ["ConfigError", "Qwen3Config", "load_config", "register_architecture", "WeightError",
           "write_model_folder", "LLM", "generate", "load_llm", "__version__"]
