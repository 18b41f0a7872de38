"""The step function and what stands on it."""
from .engine import DTYPES, Engine, Runtime, StepContext, StepError
from .plan import HostStep, StepLayout, StepPlan, build_step

__all__ = ["DTYPES", "Engine", "HostStep", "Runtime", "StepContext", "StepError", "StepLayout", "StepPlan", "build_step"]
