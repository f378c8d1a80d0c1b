"""edgerag_b200: a single-GPU inference engine for the SmolVLM / Llama text decoder on B200.

    from edgerag_b200 import Engine, SamplingParams
    engine = Engine.from_pretrained("model_dir", dtype="bfloat16")
    tokens = engine.generate([[1, 2, 3]], SamplingParams(max_new_tokens=16))

Importing the package needs no GPU (configuration, weights files, cache bookkeeping and the
scheduler are plain Python); building an ``Engine`` does, and compiles the CUDA libraries it needs
on first use.
"""

from .config import ConfigError, DecoderConfig, register_architecture
from .sampling import SamplingParams

__version__ = "0.1.0"


def __getattr__(name: str):
    if name in ("Engine", "EngineOptions", "TokenEvent"):
        from .engine import engine as _engine

        return getattr(_engine, name)
    raise AttributeError(name)


__all__ = ["ConfigError", "DecoderConfig", "Engine", "EngineOptions", "SamplingParams", "TokenEvent",
           "register_architecture"]
