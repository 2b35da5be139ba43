from .base import DefaultStepRunner, StepRunner
from .pipeline import PipelineScheduleKind, PipelineStepRunner

__all__ = ["DefaultStepRunner", "PipelineScheduleKind", "PipelineStepRunner", "StepRunner"]
