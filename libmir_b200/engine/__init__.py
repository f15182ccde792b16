from .api import (DecodeOutput, GenerationOutput, GenerationRequest, Library, Model, PrefillOutput, SamplingLogits,
                  Session)
from .context import Arena, GroupContext, StepContext
from .scheduler import PlannedEntry, Request, Scheduler
from .step import DecodeTimings, StepEntry, StepResult, StepRunner

__all__ = ["Arena", "DecodeOutput", "GenerationOutput", "GenerationRequest", "GroupContext", "Library", "Model",
           "PlannedEntry", "PrefillOutput", "Request", "SamplingLogits", "Scheduler", "Session", "StepContext",
           "DecodeTimings", "StepEntry", "StepResult", "StepRunner"]
