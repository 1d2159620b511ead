"""Training: the step object, the Trainer and its callbacks, schedules, losses, datasets."""
from .schedules import SCHEDULES, Cosine, ExponentialDecay, Lambda, Schedule, StepDecay, WarmupCosine
from .offload import GroupedOptimizer, HostOptimizer, LayerOffloader
from .run import TrainingRun
from .step import TrainStep
from .trainer import (CheckpointCallback, CsvLogger, EarlyStopping, EvaluationResult, LearningRateCallback, Metric,
                      Metrics, OutOfMemoryPolicies, Trainer, TrainerCallback, TrainingHistory)

__all__ = ["SCHEDULES", "Cosine", "ExponentialDecay", "Lambda", "Schedule", "StepDecay", "WarmupCosine", "TrainStep",
           "CheckpointCallback", "CsvLogger", "EarlyStopping", "EvaluationResult", "LearningRateCallback", "Metric",
           "Metrics", "OutOfMemoryPolicies", "Trainer", "TrainerCallback", "TrainingHistory", "GroupedOptimizer", "HostOptimizer",
           "LayerOffloader", "TrainingRun"]
