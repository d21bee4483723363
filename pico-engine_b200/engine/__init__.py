"""The step function, the generation loop above it, CUDA-graph decoding and the Engine."""
from .step import StepError, Stepper
from .generate import GenerationError, Request, generate, plan_batches, run_batch

__all__ = ["StepError", "Stepper", "GenerationError", "Request", "generate", "plan_batches", "run_batch"]
