"""A small Llama generation library for one B200: typed configuration and a registry, weights by name, layers put
together from parts, a paged cache with slots, one step function, a generation loop, sampling, and hand-written
sm_100a kernels underneath."""
from .config.registry import ConfigError, config_from_dict, load_config, register_architecture  # noqa: F401
from .sampling.options import SamplingOptions  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":  # imported on demand: it needs torch and a CUDA device
        from .engine.engine import Engine

        return Engine
    raise AttributeError(name)
