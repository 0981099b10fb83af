"""A small generation library for the Llama 3 dense decoder on one NVIDIA B200.

Everything between a request's token ids and its next token: typed configuration and
architecture registry, weights by tensor name, layers put together from parts, a paged
key/value cache with per-sequence state, one step function, a generation loop, samplers,
and hand-written sm_100a CUDA kernels underneath.  The GPU is required to run a model;
describing one (configuration, weight table, cache bookkeeping) needs none.
"""
from . import cache, config, engine, parts, weights  # noqa: F401
from .config import LlamaConfig, load_config, register_architecture

__version__ = "0.1.0"
__all__ = ["cache", "config", "engine", "parts", "weights", "LlamaConfig", "load_config", "register_architecture"]


def load(model: str, dtype: str = "bfloat16", max_tokens: int = 4096, device: int = 0, **kw):
    """Loads a model folder onto a GPU: ``load(dir).generate([[1, 2, 3]], max_new_tokens=8)``."""
    from .api import LLM
    return LLM.load(model, dtype, max_tokens, device, **kw)
