"""Trainer, flag/recipe system and the command-line application."""
from .trainer import Trainer, TrainerConfig

__all__ = ["Trainer", "TrainerConfig"]
