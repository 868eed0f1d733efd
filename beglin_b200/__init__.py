"""beglin_b200: a single-GPU inference engine for the Qwen2 dense decoder on NVIDIA B200 (sm_100a).

From a model folder (config.json and safetensors) to next-token logits and generated tokens:
typed configuration and architecture registry (`config`), weights by name (`weights`), layers put
together from parts (`parts`), a paged cache manager (`cache`), one step function with a scheduler
above it (`engine`), sampling (`sampling`) and hand-written CUDA kernels (`csrc`).
"""
__version__ = "0.1.0"

__all__ = ["Engine", "Entry", "load_config", "write_random_model"]


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "Entry":
        from .engine.batch import Entry
        return Entry
    if name == "load_config":
        from .config import load_config
        return load_config
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)
