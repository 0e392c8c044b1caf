"""Training: step function, trainer loop, checkpoints, callbacks, entry point."""

from .step import DeviceBatcher, TrainStep
from .trainer import Trainer, TrainerConfig

__all__ = ["DeviceBatcher", "TrainStep", "Trainer", "TrainerConfig"]
