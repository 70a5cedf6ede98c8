from .engine import Engine, StepError
from .context import StepContext, Workspace
from .generate import GenerationResult, Timing, generate, plan_batches, run_batches, verdict
