"""llm_singularity_b200: a small, whole, single-GPU (B200, sm_100a) inference engine."""
from .registry import known_architectures, load_config, register_architecture
from .sampling.params import SamplingParams

__all__ = ["Engine", "ModelRunner", "StepEntry", "SamplingParams", "known_architectures",
           "load_config", "register_architecture"]
__version__ = "0.1.0"


def __getattr__(name):
    # the engine pulls in torch and the kernel loader; import it on first use
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name in ("ModelRunner", "StepEntry"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
