"""llm_singularity_b200: a small, whole, single-GPU (B200, sm_100a) inference engine."""
from .registry import known_architectures, load_config, register_architecture

__all__ = ["known_architectures", "load_config", "register_architecture"]
__version__ = "0.1.0"
