from .engine import Engine, StepError
from .context import StepContext, Workspace
