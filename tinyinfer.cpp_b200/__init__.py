"""A small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

From a model folder (``config.json`` + ``model.safetensors``) to the next token:
typed configuration and registry (``config``), weights by tensor name
(``weights``), layers put together from parts (``parts``), a paged cache with
block tables and state slots (``cache``), one step function with a scheduler and
generation on top (``engine``), sampling (``sampling``) and hand-written CUDA
kernels (``csrc``, bound in ``kernels``).
"""
from .config import ConfigError, Qwen3Config, load_config, register_architecture
from .engine import Engine, LLM, StepEntry
from .sampling import SamplingParams
from .weights import WeightsError, write_random_model

__version__ = "0.1.0"

__all__ = ["ConfigError", "Engine", "LLM", "Qwen3Config", "SamplingParams", "StepEntry", "WeightsError", "load_config",
           "register_architecture", "write_random_model"]
