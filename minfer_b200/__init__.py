"""minfer_b200: a small B200-native generation library in the manner of yusiwen/minfer.

Model folder (config.json + safetensors, or seeded random weights) -> tokens in ->
logits and tokens out, on one GPU, with hand-written CUDA kernels for sm_100a.
"""
__version__ = "0.1.0"

from .config.base import ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec  # noqa: F401
from .registry import (build_part, known_architectures, read_config,  # noqa: F401
                       register_architecture, register_part)


def __getattr__(name):
    # heavier pieces are imported on first use so that `import minfer_b200` stays light
    if name in ("Model", "write_random_model"):
        from . import model
        return getattr(model, name)
    if name == "Engine":
        from .engine.step import Engine
        return Engine
    if name in ("generate", "Generator", "SamplingParams", "GenerationResult"):
        from .engine import generate as g
        return getattr(g, name)
    raise AttributeError(name)
