from .batch import SequenceStep, StepContext, StepLayout, StepPlan, context_from, plan_step
from .engine import Engine, parse_dtype
from .generate import GenerationOptions, advance, generate, plan_batches

__all__ = ["Engine", "GenerationOptions", "SequenceStep", "StepContext", "StepLayout", "StepPlan",
           "advance", "context_from", "generate", "parse_dtype", "plan_batches", "plan_step"]
