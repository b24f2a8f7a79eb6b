from .context import CacheStorage, HostStep, Scratch, StepContext, StepLayout
from .engine import Engine, EngineOptions, StepEntry, StepError, parse_dtype
