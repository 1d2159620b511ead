"""Training: the step object, the Trainer and its callbacks, schedules, losses, datasets."""
from .step import TrainStep

__all__ = ["TrainStep"]
