"""A small, whole inference engine for the Qwen2 dense decoder on one B200 (sm_100a).

    from mini_hisparse_b200 import Engine, load_model
    model = load_model("path/to/folder", device="cuda:0", dtype="bfloat16")
    engine = Engine(model, num_pages=4096)
    engine.add_request("a", [1, 2, 3], max_new_tokens=16)
    tokens = engine.run()["a"]
"""
from . import models, parts  # noqa: F401  (register the built-in parts and architectures)
from .cache import CacheConfig, CacheManager, CapacityError
from .config import ConfigError, Qwen2Config, known_architectures, register_architecture, resolve
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = [
    "CacheConfig", "CacheManager", "CapacityError", "ConfigError", "Engine", "Qwen2Config",
    "SamplingParams", "WeightError", "known_architectures", "load_model", "register_architecture",
    "resolve", "write_random_model",
]


def __getattr__(name):
    # the engine imports the kernel runtime; keep `import mini_hisparse_b200` light
    if name in ("Engine", "load_model", "make_runtime"):
        from .engine import engine as _e

        return getattr(_e, name)
    raise AttributeError(name)
