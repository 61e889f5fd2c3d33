"""Model assembly: one generic decoder built from a ModelSpec."""
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
