from .step import StepRunner, StepEntry, StepError
from .batch import StepBatch, StepContext, Workspace
from .engine import Engine, GenerationResult, StreamEvent
