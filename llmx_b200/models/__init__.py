"""Models: the generic composition and the architectures built on it."""
from .model import LayerStep, Model

__all__ = ["LayerStep", "Model"]
