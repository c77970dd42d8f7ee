from .runner import ModelRunner, StepEntry
