"""stride_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a):
config and registry, weights, parts, paged cache, one step function, scheduler,
sampling, command line, Python entry and trace replay, on hand-written CUDA kernels."""
from .engine.engine import Engine, EngineError, EngineOptions, StepEntry
from .engine.generate import LLM, GenerationResult, generate
from .engine.scheduler import GenRequest, Scheduler, SchedulerOptions, SchedulerStats, TokenEvent
from .sampling.sampler import SamplingParams

__all__ = ["Engine", "EngineError", "EngineOptions", "StepEntry", "LLM", "GenerationResult", "generate", "GenRequest",
           "Scheduler", "SchedulerOptions", "SchedulerStats", "TokenEvent", "SamplingParams"]
__version__ = "0.1.0"
