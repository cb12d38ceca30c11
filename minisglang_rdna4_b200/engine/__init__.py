from .engine import Engine, ForwardOutput, StepPlan
from .sample import BatchSamplingArgs, Sampler

__all__ = ["Engine", "ForwardOutput", "StepPlan", "BatchSamplingArgs", "Sampler"]
