"""tinyserve_b200: a small, whole, single-GPU inference engine for the dense Qwen3 decoder on
NVIDIA B200 (sm_100a), built after studying princemittalr/tinyserve.

    from tinyserve_b200 import LLM, SamplingParams
    llm = LLM.from_folder("path/to/model")            # config.json + *.safetensors
    out = llm.generate([[1, 2, 3]], max_new_tokens=8)
"""

from . import architectures  # noqa: F401  (registers the architectures)
from .cache import CacheManager
from .config import load_config, register_architecture
from .engine import LLM, Engine, Replayer
from .model import DecoderModel
from .sampling import SamplingParams
from .weights import WeightLoadError, write_random_model

__version__ = "0.1.0"

__all__ = ["CacheManager", "DecoderModel", "Engine", "LLM", "Replayer", "SamplingParams", "WeightLoadError",
           "load_config", "register_architecture", "write_random_model", "__version__"]
