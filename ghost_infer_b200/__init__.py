"""ghost-infer_b200: a small, whole model library for the Llama 3 dense decoder on one B200.

Everything between a request's tokens and its next token: typed configuration and a registry of
architectures, safetensors weights, layers put together from parts, a paged per-sequence cache, one
step function, a generation loop, sampling, and hand-written CUDA kernels for sm_100a.
"""
from .config import (ConfigError, LlamaConfig, UnknownArchitectureError, load_config, register_architecture,
                     registered_architectures)
from .config.llama_spec import build_llama_spec

from .config.barovik import BarovikConfig, build_barovik_spec

register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama_spec, replace=True)
from .config.navalorn import NavalornConfig, build_navalorn_spec

from .config.nuzinex import NuzinexConfig, build_nuzinex_spec

register_architecture("Barovik", BarovikConfig.from_dict, build_barovik_spec, replace=True)
register_architecture("Nuzinex", NuzinexConfig.from_dict, build_nuzinex_spec, replace=True)
register_architecture("Navalorn", NavalornConfig.from_dict, build_navalorn_spec, replace=True)
from .config.torutar import TorutarConfig, build_torutar_spec

register_architecture("Torutar", TorutarConfig.from_dict, build_torutar_spec, replace=True)

from .engine import Engine, Model, StepEntry  # noqa: E402
from .api import LLM  # noqa: E402
from .sampling import SamplingParams  # noqa: E402

__all__ = ["ConfigError", "LlamaConfig", "BarovikConfig", "NavalornConfig", "NuzinexConfig", "TorutarConfig", "UnknownArchitectureError", "load_config", "register_architecture",
           "registered_architectures", "Engine", "Model", "StepEntry", "LLM", "SamplingParams"]
__version__ = "0.1.0"
