"""ZeRO stage 2 (gradients and optimizer state sharded); see :mod:`maltos_b200.runtime.plugins.zero1`."""
from .zero1 import Zero2Plugin

__all__ = ["Zero2Plugin"]
