"""cpmcu_b200: a small MiniCPM4 generation library for one B200, in the manner of OpenBMB/CPM.cu.

Importing the package touches no device; kernels are compiled and loaded at first use.
"""
from .config import ConfigError, MiniCPMConfig
from .registry import Architecture, architecture, known_architectures, load_config, register_architecture
from .sampling import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM
        return LLM
    raise AttributeError(name)


__all__ = ["LLM", "ConfigError", "MiniCPMConfig", "Architecture", "architecture", "known_architectures",
           "load_config", "register_architecture", "SamplingParams"]
