"""vllm_oxide_b200: a small, whole, single-GPU inference engine for the Llama dense decoder on
B200 (sm_100a): typed configuration and registry, safetensors weights, parts, a paged cache, one
step function, a scheduler, sampling, a CLI and trace replay, over hand-written CUDA kernels."""

__version__ = "0.1.0"

from .config import EngineConfig, LlamaConfig, RopeScaling  # noqa: F401
from .errors import (EngineError, ConfigError, ShapeError, CapacityError, WeightsError,  # noqa: F401
                     WeightsFormatError, KernelError, NaNError)
