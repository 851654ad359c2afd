"""Native inference engine ("nano-inference" surface of the reference, rebuilt for B200)."""

from .engine import InferenceEngine
from .scheduler import can_schedule_any, schedule
from .types import (EngineConfig, InferenceContext, SamplingParams, SchedulerConfig, SchedulerOutput, Sequence,
                    SequenceStatus, TrainingSample)

__all__ = ["InferenceEngine", "schedule", "can_schedule_any", "EngineConfig", "InferenceContext", "SamplingParams",
           "SchedulerConfig", "SchedulerOutput", "Sequence", "SequenceStatus", "TrainingSample"]
