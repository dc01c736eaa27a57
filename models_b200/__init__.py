"""models_b200: a small model library with generation of its own for one B200 GPU.

It holds everything between a request's tokens and its next token for the Llama decoder
(LlamaForCausalLM): typed configuration and registry, weights by name, layers put together from
parts, a paged cache with a slot per sequence, one step function, a generation loop, sampling, and
trace replay -- on hand-written CUDA kernels for sm_100a.
"""

__version__ = "0.1.0"

from .config import ConfigError, LlamaConfig, config_from_dict, load_config, register_architecture
from .weights import WeightsError, load_tensors, write_random_model
from .api import CallbackStream, ModelMetadata, TextGenerationModel, TokenStream, load_model
from .engine.generation import GenerationResult, GenerationUsage, PromptCacheMetrics
from .sampling import SamplingOptions
